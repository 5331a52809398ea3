// Row-wise kernels for layers that normalise a sublayer's *result* before it joins the residual
// stream, and for models that feed a layer a weighted sum of all earlier layers' results.
//
//   norm_rows_kernel        out[o] = norm(resid[r] + delta[r]) * w, layer norm (mean taken off,
//                           variance = mean of squared deviations) or RMS norm, row selection
//   gated_norm_add_kernel   y = delta * sigmoid(gate);  x += norm(y) * w;  optionally the
//                           depth-weighted sum  sum_j mix[j] * X_j  over the kept results of all
//                           layers so far, and a copy of the outgoing row in the compute dtype
//                           for the projection that reads it next
//   xielu_kernel            the two-branch quadratic / exponential activation
//   softcap_kernel          cap * tanh(v / cap) on float32 logits
//   cast_rows_kernel        float32 rows -> compute dtype
//
// Statistics, sigmoids, the residual sum and the depth-weighted sum are float32 whatever the
// storage type.  Every sum has a fixed order that depends on the row length only, so a row's
// result does not depend on what else is in the step.
#include "common.cuh"

namespace vx {

constexpr int RN_MAX_PER_THREAD = 8;

__device__ __forceinline__ float sigmoid_f32(float v) { return 1.0f / (1.0f + expf(-v)); }
// The gate of a row whose sublayer result and gate logits are bfloat16: the fast exponential and
// division are exact far beyond what the operands carry.  float32 rows keep the accurate form.
template <typename T>
__device__ __forceinline__ float gate_sigmoid(float v) { return sigmoid_f32(v); }
template <>
__device__ __forceinline__ float gate_sigmoid<__nv_bfloat16>(float v) { return __fdividef(1.0f, 1.0f + __expf(-v)); }

// Mean (0 when `center` is off) and 1 / sqrt(mean((v - mean)^2) + eps) of a row given by
// `value(i)`; two passes over the row, as the definition says.  `vals` caches the row when it
// fits (hidden <= RN_MAX_PER_THREAD * blockDim.x).
template <typename F>
__device__ __forceinline__ void row_statistics(F value, int hidden, int center, float eps, bool cached,
                                               float (&vals)[RN_MAX_PER_THREAD], float* scratch, float& mean,
                                               float& inv) {
  float s = 0.f;
  if (cached) {
#pragma unroll
    for (int j = 0; j < RN_MAX_PER_THREAD; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      vals[j] = i < hidden ? value(i) : 0.f;
      s += vals[j];
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) s += value(i);
  }
  mean = 0.f;
  if (center) mean = block_sum(s, scratch) / (float)hidden;
  float ss = 0.f;
  if (cached) {
#pragma unroll
    for (int j = 0; j < RN_MAX_PER_THREAD; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      const float d = i < hidden ? vals[j] - mean : 0.f;
      ss += d * d;
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      const float d = value(i) - mean;
      ss += d * d;
    }
  }
  ss = block_sum(ss, scratch);
  inv = 1.0f / sqrtf(ss / (float)hidden + eps);
}

// ---------------------------------------------------------------------------------------------
// out[o] = norm(resid[r] + delta[r]) * weight, r = rows ? rows[o] : o.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void norm_rows_kernel(float* __restrict__ resid, const T* __restrict__ delta,
                                 const float* __restrict__ weight, float eps, int center, T* __restrict__ out,
                                 const int* __restrict__ rows, int hidden, int write_resid) {
  __shared__ float scratch[32];
  allow_dependents();
  grid_dependency_wait();
  const int o = blockIdx.x;
  const int r = rows ? rows[o] : o;
  float* x = resid + (size_t)r * hidden;
  const T* d = delta ? delta + (size_t)r * hidden : nullptr;
  auto value = [&](int i) { return d ? x[i] + to_float(d[i]) : x[i]; };
  const bool cached = hidden <= RN_MAX_PER_THREAD * (int)blockDim.x;
  float vals[RN_MAX_PER_THREAD], mean, inv;
  row_statistics(value, hidden, center, eps, cached, vals, scratch, mean, inv);
  T* y = out + (size_t)o * hidden;
  if (cached) {
#pragma unroll
    for (int j = 0; j < RN_MAX_PER_THREAD; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      if (i < hidden) {
        if (write_resid && d) x[i] = vals[j];
        y[i] = from_float<T>((vals[j] - mean) * inv * weight[i]);
      }
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      const float v = value(i);
      if (write_resid && d) x[i] = v;
      y[i] = from_float<T>((v - mean) * inv * weight[i]);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// A sublayer's result joins the stream:
//   y        = delta[r] * sigmoid(gate[r])            (gate null: y = delta[r])
//              delta32 given instead of delta: the result lies in a float32 buffer into which a
//              projection has added its shares (y uses delta32[r] + delta_bias), and the rows
//              read are set to zero again, so that the next sums start from nothing
//   x        = resid_in[r] + norm(y) * weight         -> resid_out[r]
//   outgoing = x                                      (mix_terms == 0)
//            = sum_{j < mix_terms - 1} mix_w[j] * hist[j][r]  +  mix_w[mix_terms - 1] * x
//                                                      -> mix_out[r]
//   lowp_out[r] = outgoing in the compute dtype (null: not written)
// hist[j] = hist + j * hist_stride holds the kept rows of earlier results, [*, hidden] each.
// resid_in may equal resid_out.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void gated_norm_add_kernel(const float* resid_in, float* resid_out, const T* __restrict__ delta,
                                      long long delta_ld, const T* __restrict__ gate, long long gate_ld,
                                      const float* __restrict__ weight, float eps, int center,
                                      T* __restrict__ lowp_out, const float* __restrict__ hist,
                                      long long hist_stride, const float* __restrict__ mix_w, int mix_terms,
                                      float* __restrict__ mix_out, int hidden, float* __restrict__ delta32,
                                      long long delta32_ld, const float* __restrict__ delta_bias) {
  __shared__ float scratch[32];
  allow_dependents();
  grid_dependency_wait();
  const int r = blockIdx.x;
  const T* d = delta ? delta + (size_t)r * delta_ld : nullptr;
  float* d32 = delta32 ? delta32 + (size_t)r * delta32_ld : nullptr;
  const T* g = gate ? gate + (size_t)r * gate_ld : nullptr;
  auto value = [&](int i) {
    float v = d32 ? d32[i] : to_float(d[i]);
    if (delta_bias) v += delta_bias[i];
    return g ? v * sigmoid_f32(to_float(g[i])) : v;
  };
  const bool cached = hidden <= RN_MAX_PER_THREAD * (int)blockDim.x;
  float vals[RN_MAX_PER_THREAD], mean, inv;
  row_statistics(value, hidden, center, eps, cached, vals, scratch, mean, inv);
  const float* xin = resid_in + (size_t)r * hidden;
  float* xout = resid_out + (size_t)r * hidden;
  auto finish = [&](int i, float v) {
    const float x = xin[i] + (v - mean) * inv * weight[i];
    xout[i] = x;
    float outgoing = x;
    if (mix_terms > 0) {
      float acc = 0.f;
      for (int j = 0; j + 1 < mix_terms; ++j)
        acc = fmaf(mix_w[j], hist[(size_t)j * hist_stride + (size_t)r * hidden + i], acc);
      outgoing = fmaf(mix_w[mix_terms - 1], x, acc);
      mix_out[(size_t)r * hidden + i] = outgoing;
    }
    if (lowp_out) lowp_out[(size_t)r * hidden + i] = from_float<T>(outgoing);
    if (d32) d32[i] = 0.f;  // the sums' buffer is handed back empty
  };
  if (cached) {
#pragma unroll
    for (int j = 0; j < RN_MAX_PER_THREAD; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      if (i < hidden) finish(i, vals[j]);
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) finish(i, value(i));
  }
}

// ---------------------------------------------------------------------------------------------
// xIELU: z > 0: a_pos z^2 + z / 2;  z <= 0: a_neg (exp(z) - 1 - z) + z / 2, on [T, n] read with a
// row pitch (the columns may be part of a wider projection) and written densely.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void xielu_kernel(const T* __restrict__ in, long long in_ld, T* __restrict__ out, long long total,
                             int n, float a_pos, float a_neg) {
  allow_dependents();
  grid_dependency_wait();
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
    const long long t = idx / n;
    const int i = (int)(idx - t * n);
    const float z = to_float(in[t * in_ld + i]);
    const float v = z > 0.f ? fmaf(a_pos * z, z, 0.5f * z) : fmaf(a_neg, expm1f(z) - z, 0.5f * z);
    out[idx] = from_float<T>(v);
  }
}

__global__ void softcap_kernel(float* __restrict__ values, long long total, float cap) {
  allow_dependents();
  grid_dependency_wait();
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride)
    values[idx] = cap * tanhf(values[idx] / cap);
}

__global__ void cast_rows_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out, long long total) {
  allow_dependents();
  grid_dependency_wait();
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride)
    out[idx] = __float2bfloat16_rn(in[idx]);
}

// ---------------------------------------------------------------------------------------------
// Vector forms, for rows of whole chunks of four elements that start on the boundaries a chunk's
// load needs (16 bytes in float32, 8 in bfloat16): a thread keeps up to GV_CHUNKS chunks in
// registers across the two reductions: four warps a row and up to four chunks a thread (rows of
// up to 2,048 elements), or eight warps and up to eight chunks (up to 8,192).  The same formulas;
// the order of a row's sums depends on the row's length only.
// ---------------------------------------------------------------------------------------------
constexpr int GV_CHUNKS = 8;

template <typename T>
__device__ __forceinline__ float4 load4(const T* p);
template <>
__device__ __forceinline__ float4 load4<float>(const float* p) {
  return *reinterpret_cast<const float4*>(p);
}
template <>
__device__ __forceinline__ float4 load4<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
template <typename T>
__device__ __forceinline__ void store4(T* p, float4 v);
template <>
__device__ __forceinline__ void store4<float>(float* p, float4 v) {
  *reinterpret_cast<float4*>(p) = v;
}
template <>
__device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, float4 v) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<const uint32_t*>(&a);
  raw.y = *reinterpret_cast<const uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = raw;
}

template <typename T, int CHUNKS>
__global__ void gated_norm_add_vec_kernel(const float* resid_in, float* resid_out, const T* __restrict__ delta,
                                          long long delta_ld, const T* __restrict__ gate, long long gate_ld,
                                          const float* __restrict__ weight, float eps, int center,
                                          T* __restrict__ lowp_out, const float* __restrict__ hist,
                                          long long hist_stride, const float* __restrict__ mix_w, int mix_terms,
                                          float* __restrict__ mix_out, int hidden, float* __restrict__ delta32,
                                          long long delta32_ld, const float* __restrict__ delta_bias) {
  __shared__ float scratch[32];
  allow_dependents();
  grid_dependency_wait();
  const int r = blockIdx.x;
  const int chunks = hidden / 4;
  const T* d = delta ? delta + (size_t)r * delta_ld : nullptr;
  float* d32 = delta32 ? delta32 + (size_t)r * delta32_ld : nullptr;
  const T* g = gate ? gate + (size_t)r * gate_ld : nullptr;
  const size_t row = (size_t)r * hidden;
  // Everything the row needs is asked for before the first reduction: the sublayer's result and
  // its gate, and the stream's rows and the weight that are only used after the second one.
  float4 y[CHUNKS], e[CHUNKS], xin[CHUNKS], wv[CHUNKS];
#pragma unroll
  for (int j = 0; j < CHUNKS; ++j) {
    const int c = threadIdx.x + j * blockDim.x;
    y[j] = e[j] = xin[j] = wv[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c < chunks) {
      y[j] = d32 ? *reinterpret_cast<const float4*>(d32 + 4 * c) : load4<T>(d + 4 * c);
      if (delta_bias) {
        const float4 b = __ldg(reinterpret_cast<const float4*>(delta_bias + 4 * c));
        y[j].x += b.x;
        y[j].y += b.y;
        y[j].z += b.z;
        y[j].w += b.w;
      }
      if (g) e[j] = load4<T>(g + 4 * c);
      xin[j] = *reinterpret_cast<const float4*>(resid_in + row + 4 * c);
      wv[j] = __ldg(reinterpret_cast<const float4*>(weight + 4 * c));
    }
  }
  if (d32) {  // the sums' buffer is handed back empty
#pragma unroll
    for (int j = 0; j < CHUNKS; ++j) {
      const int c = threadIdx.x + j * blockDim.x;
      if (c < chunks) *reinterpret_cast<float4*>(d32 + 4 * c) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < CHUNKS; ++j) {
    if (g) {
      y[j].x *= gate_sigmoid<T>(e[j].x);
      y[j].y *= gate_sigmoid<T>(e[j].y);
      y[j].z *= gate_sigmoid<T>(e[j].z);
      y[j].w *= gate_sigmoid<T>(e[j].w);
    }
    s += (y[j].x + y[j].y) + (y[j].z + y[j].w);
  }
  float mean = 0.f;
  if (center) mean = block_sum(s, scratch) / (float)hidden;
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < CHUNKS; ++j) {
    const int c = threadIdx.x + j * blockDim.x;
    if (c < chunks) {
      const float a = y[j].x - mean, b = y[j].y - mean, p = y[j].z - mean, q = y[j].w - mean;
      ss += (a * a + b * b) + (p * p + q * q);
    }
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
  float4 x[CHUNKS];
#pragma unroll
  for (int j = 0; j < CHUNKS; ++j) {
    x[j].x = xin[j].x + (y[j].x - mean) * inv * wv[j].x;
    x[j].y = xin[j].y + (y[j].y - mean) * inv * wv[j].y;
    x[j].z = xin[j].z + (y[j].z - mean) * inv * wv[j].z;
    x[j].w = xin[j].w + (y[j].w - mean) * inv * wv[j].w;
    const int c = threadIdx.x + j * blockDim.x;
    if (c < chunks) *reinterpret_cast<float4*>(resid_out + row + 4 * c) = x[j];
  }
  if (mix_terms > 0) {
    // One earlier result at a time, all of the thread's chunks of it asked for at once.
    float4 acc[CHUNKS];
#pragma unroll
    for (int j = 0; j < CHUNKS; ++j) acc[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = 0; k + 1 < mix_terms; ++k) {
      const float m = mix_w[k];
      const float* src = hist + (size_t)k * hist_stride + row;
      float4 v[CHUNKS];
#pragma unroll
      for (int j = 0; j < CHUNKS; ++j) {
        const int c = threadIdx.x + j * blockDim.x;
        v[j] = c < chunks ? *reinterpret_cast<const float4*>(src + 4 * c) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int j = 0; j < CHUNKS; ++j) {
        acc[j].x = fmaf(m, v[j].x, acc[j].x);
        acc[j].y = fmaf(m, v[j].y, acc[j].y);
        acc[j].z = fmaf(m, v[j].z, acc[j].z);
        acc[j].w = fmaf(m, v[j].w, acc[j].w);
      }
    }
    const float m = mix_w[mix_terms - 1];
#pragma unroll
    for (int j = 0; j < CHUNKS; ++j) {
      x[j] = make_float4(fmaf(m, x[j].x, acc[j].x), fmaf(m, x[j].y, acc[j].y), fmaf(m, x[j].z, acc[j].z),
                         fmaf(m, x[j].w, acc[j].w));
      const int c = threadIdx.x + j * blockDim.x;
      if (c < chunks) *reinterpret_cast<float4*>(mix_out + row + 4 * c) = x[j];
    }
  }
  if (lowp_out) {
#pragma unroll
    for (int j = 0; j < CHUNKS; ++j) {
      const int c = threadIdx.x + j * blockDim.x;
      if (c < chunks) store4<T>(lowp_out + row + 4 * c, x[j]);
    }
  }
}

template <typename T, int CHUNKS>
static void launch_gated_norm_add_vec(int block, const float* resid_in, float* resid_out, const void* delta,
                                      long long delta_ld, const void* gate, long long gate_ld, const float* weight,
                                      float eps, int center, void* lowp_out, const float* hist, long long hist_stride,
                                      const float* mix_w, int mix_terms, float* mix_out, int num_rows, int hidden,
                                      float* delta32, long long delta32_ld, const float* delta_bias,
                                      cudaStream_t stream) {
  launch_pdl(gated_norm_add_vec_kernel<T, CHUNKS>, dim3(num_rows), dim3(block), 0, stream, resid_in, resid_out,
             (const T*)delta, delta_ld, (const T*)gate, gate_ld, weight, eps, center, (T*)lowp_out, hist, hist_stride,
             mix_w, mix_terms, mix_out, hidden, delta32, delta32_ld, delta_bias);
}

// Eight (bfloat16) or four (float32) activations a thread; n, the row pitch and the pointers allow
// 16-byte accesses.
// The negative branch needs exp(z) - 1 - z.  float32 keeps expm1f (no cancellation near 0); in
// bfloat16 the fast exponential's absolute error of about 1e-7 is far below what the result is
// rounded to, and the accurate form would make the kernel compute-bound.
template <typename T>
__device__ __forceinline__ float exp_minus_one(float z);
template <>
__device__ __forceinline__ float exp_minus_one<float>(float z) { return expm1f(z); }
template <>
__device__ __forceinline__ float exp_minus_one<__nv_bfloat16>(float z) { return __expf(z) - 1.0f; }

template <typename T>
__global__ void xielu_vec_kernel(const T* __restrict__ in, long long in_ld, T* __restrict__ out, long long vectors,
                                 int per_row, float a_pos, float a_neg) {
  constexpr int W = 16 / (int)sizeof(T);
  allow_dependents();
  grid_dependency_wait();
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < vectors; idx += stride) {
    const long long t = idx / per_row;
    const int c = (int)(idx - t * per_row);
    const T* src = in + t * in_ld + (size_t)c * W;
    T* dst = out + idx * W;
#pragma unroll
    for (int half = 0; half < W / 4; ++half) {
      float4 z = load4<T>(src + 4 * half);
      float* e = reinterpret_cast<float*>(&z);
#pragma unroll
      for (int i = 0; i < 4; ++i)
        e[i] = e[i] > 0.f ? fmaf(a_pos * e[i], e[i], 0.5f * e[i]) : fmaf(a_neg, exp_minus_one<T>(e[i]) - e[i], 0.5f * e[i]);
      store4<T>(dst + 4 * half, z);
    }
  }
}

static bool aligned_to(const void* p, int bytes) { return (reinterpret_cast<uintptr_t>(p) & (uintptr_t)(bytes - 1)) == 0; }

static int row_threads(int hidden) {
  int threads = ((hidden + 3) / 4 + 31) / 32 * 32;
  return threads < 64 ? 64 : (threads > 1024 ? 1024 : threads);
}

static int flat_blocks(long long total, int threads) {
  long long blocks = (total + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  return (int)blocks;
}

}  // namespace vx

using namespace vx;

VX_API int vx_norm_rows(float* resid, const void* delta, const float* weight, float eps, int center, void* out,
                        int dtype, const int* rows, int num_out_rows, int hidden, int write_resid,
                        cudaStream_t stream) {
  if (num_out_rows <= 0) return 0;
  const int threads = row_threads(hidden);
  if (dtype == VX_DTYPE_F32)
    launch_pdl(norm_rows_kernel<float>, dim3(num_out_rows), dim3(threads), 0, stream, resid, (const float*)delta,
               weight, eps, center, (float*)out, rows, hidden, write_resid);
  else
    launch_pdl(norm_rows_kernel<__nv_bfloat16>, dim3(num_out_rows), dim3(threads), 0, stream, resid,
               (const __nv_bfloat16*)delta, weight, eps, center, (__nv_bfloat16*)out, rows, hidden, write_resid);
  return (int)cudaGetLastError();
}

VX_API int vx_gated_norm_add(const float* resid_in, float* resid_out, const void* delta, long long delta_ld,
                             const void* gate, long long gate_ld, const float* weight, float eps, int center,
                             void* lowp_out, int dtype, const float* hist, long long hist_stride,
                             const float* mix_w, int mix_terms, float* mix_out, int num_rows, int hidden,
                             float* delta32, long long delta32_ld, const float* delta_bias, cudaStream_t stream) {
  if (num_rows <= 0) return 0;
  if ((delta == nullptr) == (delta32 == nullptr)) return (int)cudaErrorInvalidValue;
  if (mix_terms > 0 && (mix_w == nullptr || mix_out == nullptr || (mix_terms > 1 && hist == nullptr)))
    return (int)cudaErrorInvalidValue;
  // Whole chunks of four that every pointer and pitch lets a thread load at once.
  const int unit = dtype == VX_DTYPE_F32 ? 16 : 8, per = dtype == VX_DTYPE_F32 ? 4 : 2;
  const bool vec = hidden % 4 == 0 && hidden / 4 <= 256 * GV_CHUNKS && aligned_to(resid_in, 16) && aligned_to(resid_out, 16) &&
                   aligned_to(weight, 16) &&
                   (delta32 != nullptr ? (aligned_to(delta32, 16) && delta32_ld % 4 == 0)
                                       : (aligned_to(delta, unit) && (delta_ld * per) % unit == 0)) &&
                   (delta_bias == nullptr || aligned_to(delta_bias, 16)) &&
                   (gate == nullptr || (aligned_to(gate, unit) && (gate_ld * per) % unit == 0)) &&
                   (lowp_out == nullptr || aligned_to(lowp_out, unit)) &&
                   (mix_terms == 0 || (aligned_to(mix_out, 16) && (hist == nullptr || (aligned_to(hist, 16) && hist_stride % 4 == 0))));
  if (vec) {
    const int chunks = hidden / 4;
    const int block = chunks <= 128 * 4 ? 128 : 256;
    const int per = (chunks + block - 1) / block;
#define VX_GNA(T, C)                                                                                              \
  launch_gated_norm_add_vec<T, C>(block, resid_in, resid_out, delta, delta_ld, gate, gate_ld, weight, eps, center, \
                                  lowp_out, hist, hist_stride, mix_w, mix_terms, mix_out, num_rows, hidden, delta32,    \
                                  delta32_ld, delta_bias, stream)
    if (dtype == VX_DTYPE_F32) {
      if (per <= 1) VX_GNA(float, 1); else if (per <= 2) VX_GNA(float, 2); else if (per <= 4) VX_GNA(float, 4); else VX_GNA(float, 8);
    } else {
      if (per <= 1) VX_GNA(__nv_bfloat16, 1); else if (per <= 2) VX_GNA(__nv_bfloat16, 2);
      else if (per <= 4) VX_GNA(__nv_bfloat16, 4); else VX_GNA(__nv_bfloat16, 8);
    }
#undef VX_GNA
    return (int)cudaGetLastError();
  }
  const int threads = row_threads(hidden);
  if (dtype == VX_DTYPE_F32)
    launch_pdl(gated_norm_add_kernel<float>, dim3(num_rows), dim3(threads), 0, stream, resid_in, resid_out,
               (const float*)delta, delta_ld, (const float*)gate, gate_ld, weight, eps, center, (float*)lowp_out,
               hist, hist_stride, mix_w, mix_terms, mix_out, hidden, delta32, delta32_ld, delta_bias);
  else
    launch_pdl(gated_norm_add_kernel<__nv_bfloat16>, dim3(num_rows), dim3(threads), 0, stream, resid_in, resid_out,
               (const __nv_bfloat16*)delta, delta_ld, (const __nv_bfloat16*)gate, gate_ld, weight, eps, center,
               (__nv_bfloat16*)lowp_out, hist, hist_stride, mix_w, mix_terms, mix_out, hidden, delta32, delta32_ld,
               delta_bias);
  return (int)cudaGetLastError();
}

VX_API int vx_xielu(const void* in, long long in_ld, void* out, int dtype, int num_rows, int n, float a_pos,
                    float a_neg, cudaStream_t stream) {
  const long long total = (long long)num_rows * n;
  if (total <= 0) return 0;
  const int width = dtype == VX_DTYPE_F32 ? 4 : 8;
  if (n % width == 0 && in_ld % width == 0 && aligned_to(in, 16) && aligned_to(out, 16)) {
    const long long vectors = total / width;
    if (dtype == VX_DTYPE_F32)
      launch_pdl(xielu_vec_kernel<float>, dim3(flat_blocks(vectors, 256)), dim3(256), 0, stream, (const float*)in, in_ld,
                 (float*)out, vectors, n / width, a_pos, a_neg);
    else
      launch_pdl(xielu_vec_kernel<__nv_bfloat16>, dim3(flat_blocks(vectors, 256)), dim3(256), 0, stream,
                 (const __nv_bfloat16*)in, in_ld, (__nv_bfloat16*)out, vectors, n / width, a_pos, a_neg);
    return (int)cudaGetLastError();
  }
  if (dtype == VX_DTYPE_F32)
    launch_pdl(xielu_kernel<float>, dim3(flat_blocks(total, 256)), dim3(256), 0, stream, (const float*)in, in_ld,
               (float*)out, total, n, a_pos, a_neg);
  else
    launch_pdl(xielu_kernel<__nv_bfloat16>, dim3(flat_blocks(total, 256)), dim3(256), 0, stream,
               (const __nv_bfloat16*)in, in_ld, (__nv_bfloat16*)out, total, n, a_pos, a_neg);
  return (int)cudaGetLastError();
}

VX_API int vx_softcap(float* values, long long total, float cap, cudaStream_t stream) {
  if (total <= 0) return 0;
  if (!(cap > 0.f)) return (int)cudaErrorInvalidValue;
  launch_pdl(softcap_kernel, dim3(flat_blocks(total, 256)), dim3(256), 0, stream, values, total, cap);
  return (int)cudaGetLastError();
}

VX_API int vx_cast_f32_to_bf16(const float* in, void* out, long long total, cudaStream_t stream) {
  if (total <= 0) return 0;
  launch_pdl(cast_rows_kernel, dim3(flat_blocks(total, 256)), dim3(256), 0, stream, in, (__nv_bfloat16*)out, total);
  return (int)cudaGetLastError();
}
