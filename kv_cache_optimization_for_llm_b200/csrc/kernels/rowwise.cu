// Row-wise kernels for layers that norm a branch's output before it joins the residual
// stream: one kernel does  post-norm of the branch -> residual add -> pre-norm of the next
// sublayer,  with layer norm or RMS norm on either side; and the activation kernel of a
// gated feed-forward with biases.  Statistics, the residual and the activation's
// arithmetic are float32 whatever the activations' type.
#include "common.cuh"

enum NormKind { NORM_NONE = 0, NORM_LAYER = 1, NORM_RMS = 2 };

constexpr int kRowThreads = 256;

// Sum over the block; every thread gets the total, added in an order that depends on the
// block size only.  `part` holds one float per warp and may be reused right after.
__device__ __forceinline__ float row_block_sum(float v, float* part) {
  v = warp_sum(v);
  __syncthreads();               // the previous use of `part` is over
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
  const int nw = blockDim.x >> 5;
  for (int i = 0; i < nw; ++i) t += part[i];
  return t;
}

// mean and 1/sqrt(var + eps) (layer norm) or 0 and 1/sqrt(mean square + eps) (RMS norm) of the
// row held in shared memory.  The variance is the mean of the squared deviations from the mean,
// taken in a second pass.
__device__ __forceinline__ void row_stats(const float* row, int H, int kind, float eps, float* part,
                                          float& mean, float& rstd) {
  mean = 0.f;
  if (kind == NORM_LAYER) {
    float s = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) s += row[i];
    mean = row_block_sum(s, part) / (float)H;
  }
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float d = row[i] - mean;
    ss += d * d;
  }
  rstd = 1.0f / sqrtf(row_block_sum(ss, part) / (float)H + eps);
}

// For output row b (token row t = rows ? rows[b] : b):
//   d = delta[t] + delta_bias                       (when a branch output is pending)
//   v = resid[t] + post(d) * post_w                 post: layer norm, RMS norm or identity
//   resid[t] = v                                    (only when every row is produced: rows == null)
//   out[b] = pre(v) * pre_w                         pre: layer norm or RMS norm; NORM_NONE: v itself in the
//                                                   activations' type when out is given, else no output
template <typename T>
__global__ void __launch_bounds__(kRowThreads)
add_norm_kernel(float* __restrict__ resid, const T* __restrict__ delta, const float* __restrict__ delta_bias,
                const float* __restrict__ post_w, int post_kind, float post_eps,
                const float* __restrict__ pre_w, int pre_kind, float pre_eps,
                T* __restrict__ out, const int* __restrict__ rows, int H) {
  extern __shared__ float row[];
  __shared__ float part[32];
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.x;
  const size_t src = (size_t)(rows ? rows[b] : b) * H;
  float mean, rstd;
  if (delta != nullptr) {
    for (int i = threadIdx.x; i < H; i += blockDim.x)
      row[i] = to_f32(delta[src + i]) + (delta_bias ? delta_bias[i] : 0.f);
    __syncthreads();
    if (post_kind != NORM_NONE) {
      row_stats(row, H, post_kind, post_eps, part, mean, rstd);
    } else {
      mean = 0.f; rstd = 1.f;
    }
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      const float v = resid[src + i] + (row[i] - mean) * rstd * (post_w ? post_w[i] : 1.f);
      row[i] = v;
      if (!rows) resid[src + i] = v;
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) row[i] = resid[src + i];
  }
  T* o = out + (size_t)b * H;
  if (pre_kind == NORM_NONE) {
    // a sublayer that reads the stream itself: the thread that made an element hands it on
    if (out != nullptr)
      for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = from_f32<T>(row[i]);
    return;
  }
  __syncthreads();
  row_stats(row, H, pre_kind, pre_eps, part, mean, rstd);
  for (int i = threadIdx.x; i < H; i += blockDim.x)
    o[i] = from_f32<T>((row[i] - mean) * rstd * (pre_w ? pre_w[i] : 1.f));
}

KVB_EXPORT int kvb_add_norm(float* resid, const void* delta, const float* delta_bias, const float* post_w,
                            int post_kind, float post_eps, const float* pre_w, int pre_kind, float pre_eps,
                            void* out, const int* rows, int n_out_rows, int H, int dtype, cudaStream_t stream) {
  if (n_out_rows <= 0) return 0;
  if (post_kind < 0 || post_kind > 2 || pre_kind < 0 || pre_kind > 2) return KVB_ERR_BAD_SIZE;
  const size_t smem = (size_t)H * sizeof(float);
  if (smem > 200 * 1024) return KVB_ERR_BAD_SIZE;
  KVB_DISPATCH_DTYPE(dtype, T, {
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(add_norm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
    }
    kvb_launch(add_norm_kernel<T>, dim3(n_out_rows), dim3(kRowThreads), smem, stream, resid, (const T*)delta,
               delta_bias, post_w, post_kind, post_eps, pre_w, pre_kind, pre_eps, (T*)out, rows, H);
  });
  return kvb_launch_result();
}

// ---------------------------------------------------------------- act(gate + b) * (up + b)
enum ActKind { ACT_SILU = 0, ACT_GELU_TANH = 1 };

__device__ __forceinline__ float act_apply(float z, int kind) {
  if (kind == ACT_GELU_TANH) {
    const float c = 0.7978845608028654f;   // sqrt(2 / pi)
    return 0.5f * z * (1.0f + tanhf(c * (z + 0.044715f * z * z * z)));
  }
  return z / (1.0f + expf(-z));
}

// gu [T, 2 I] holds a row's gate features, then its up features; the biases (float32, may be
// null) are [2 I] in the same order.  out[t, i] = act(gate + b) * (up + b).
template <typename T>
__global__ void bias_act_mul_kernel(const T* __restrict__ gu, const float* __restrict__ bias, T* __restrict__ out,
                                    int I, int kind, size_t total) {
  pdl_trigger();
  pdl_wait();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / I;
    const int i = (int)(idx - t * I);
    float g = to_f32(gu[t * 2 * I + i]), u = to_f32(gu[t * 2 * I + I + i]);
    if (bias) { g += bias[i]; u += bias[I + i]; }
    out[idx] = from_f32<T>(act_apply(g, kind) * u);
  }
}

// bfloat16 rows whose halves are multiples of 8 wide: eight elements per thread, 16-byte accesses.
__global__ void bias_act_mul_bf16x8_kernel(const __nv_bfloat16* __restrict__ gu, const float* __restrict__ bias,
                                           __nv_bfloat16* __restrict__ out, int I, int kind, size_t groups) {
  pdl_trigger();
  pdl_wait();
  const int gpr = I >> 3;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < groups;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / gpr;
    const int i = (int)(idx - t * gpr) << 3;
    const uint4 g = *reinterpret_cast<const uint4*>(gu + t * 2 * I + i);
    const uint4 u = *reinterpret_cast<const uint4*>(gu + t * 2 * I + I + i);
    const unsigned gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
    unsigned ow[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float g0 = __uint_as_float(gw[k] << 16), g1 = __uint_as_float(gw[k] & 0xffff0000u);
      float u0 = __uint_as_float(uw[k] << 16), u1 = __uint_as_float(uw[k] & 0xffff0000u);
      if (bias) {
        g0 += bias[i + 2 * k]; g1 += bias[i + 2 * k + 1];
        u0 += bias[I + i + 2 * k]; u1 += bias[I + i + 2 * k + 1];
      }
      __nv_bfloat162 v = __floats2bfloat162_rn(act_apply(g0, kind) * u0, act_apply(g1, kind) * u1);
      ow[k] = *reinterpret_cast<unsigned*>(&v);
    }
    *reinterpret_cast<uint4*>(out + t * I + i) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
  }
}

KVB_EXPORT int kvb_bias_act_mul(const void* gu, const float* bias, void* out, int T_, int I, int kind, int dtype,
                                cudaStream_t stream) {
  if (T_ <= 0) return 0;
  if (I < 1 || kind < 0 || kind > 1) return KVB_ERR_BAD_SIZE;
  if (dtype == KVB_BF16 && I % 8 == 0 && (reinterpret_cast<uintptr_t>(gu) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
    const size_t groups = (size_t)T_ * (I / 8);
    const size_t want8 = (groups + 255) / 256;
    const int blocks8 = (int)(want8 < (size_t)kvb_sm_count() * 16 ? want8 : (size_t)kvb_sm_count() * 16);
    kvb_launch(bias_act_mul_bf16x8_kernel, dim3(blocks8), dim3(256), 0, stream, (const __nv_bfloat16*)gu, bias,
               (__nv_bfloat16*)out, I, kind, groups);
    return kvb_launch_result();
  }
  const size_t total = (size_t)T_ * I;
  const size_t want = (total + 255) / 256;
  const int blocks = (int)(want < (size_t)kvb_sm_count() * 16 ? want : (size_t)kvb_sm_count() * 16);
  KVB_DISPATCH_DTYPE(dtype, T, (kvb_launch(bias_act_mul_kernel<T>, dim3(blocks), dim3(256), 0, stream, (const T*)gu,
                                            bias, (T*)out, I, kind, total)));
  return kvb_launch_result();
}

// ---------------------------------------------------------------- logits: a factor, then a soft cap
// x[i] <- cap * tanh(x[i] * scale / cap) in place on float32 (cap 0: only the factor).
__global__ void scale_softcap_kernel(float* __restrict__ x, float scale, float cap, size_t total) {
  pdl_trigger();
  pdl_wait();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const float z = x[idx] * scale;
    x[idx] = cap > 0.f ? cap * tanhf(z / cap) : z;
  }
}

KVB_EXPORT int kvb_scale_softcap(float* x, size_t total, float scale, float cap, cudaStream_t stream) {
  if (total == 0) return 0;
  if (cap < 0.f) return KVB_ERR_BAD_SIZE;
  const size_t want = (total + 255) / 256;
  const int blocks = (int)(want < (size_t)kvb_sm_count() * 16 ? want : (size_t)kvb_sm_count() * 16);
  kvb_launch(scale_softcap_kernel, dim3(blocks), dim3(256), 0, stream, x, scale, cap, total);
  return kvb_launch_result();
}

// ---------------------------------------------------------------- tanh of a slice of columns
// out[t, i] = tanh(in[t * ld + i]) for i < n: the middle of a low-rank branch whose first
// product is part of a wider one.
template <typename T>
__global__ void tanh_slice_kernel(const T* __restrict__ in, int ld, T* __restrict__ out, int n, size_t total) {
  pdl_trigger();
  pdl_wait();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / n;
    const int i = (int)(idx - t * n);
    out[idx] = from_f32<T>(tanhf(to_f32(in[t * ld + i])));
  }
}

KVB_EXPORT int kvb_tanh_slice(const void* in, int ld, void* out, int T_, int n, int dtype, cudaStream_t stream) {
  if (T_ <= 0 || n <= 0) return 0;
  const size_t total = (size_t)T_ * n;
  const size_t want = (total + 255) / 256;
  const int blocks = (int)(want < (size_t)kvb_sm_count() * 16 ? want : (size_t)kvb_sm_count() * 16);
  KVB_DISPATCH_DTYPE(dtype, T, (kvb_launch(tanh_slice_kernel<T>, dim3(blocks), dim3(256), 0, stream, (const T*)in, ld,
                                            (T*)out, n, total)));
  return kvb_launch_result();
}

// ---------------------------------------------------------------- several summands join the residual, then a norm
// For output row b (token row t = rows ? rows[b] : b):
//   v = resid[t] + d1[t] + d2[t] + e[t] + vec        every summand optional: two branch outputs (a layer whose
//                                                     sublayers read the same normed input), float32 rows (the
//                                                     embedding's output re-entering), one float32 vector for all rows
//   resid[t] = v                                      (only when every row is produced: rows == null)
//   out[b] = v / sqrt(mean(v^2) + eps) * w            NORM_RMS; NORM_NONE: no output.  out is float32 when out_f32.
template <typename T>
__global__ void __launch_bounds__(kRowThreads)
join_norm_kernel(float* __restrict__ resid, const T* __restrict__ d1, const T* __restrict__ d2,
                 const float* __restrict__ e, const float* __restrict__ vec, const float* __restrict__ w, int kind,
                 float eps, void* __restrict__ out, int out_f32, const int* __restrict__ rows, int H) {
  extern __shared__ float row[];
  __shared__ float part[32];
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.x;
  const size_t src = (size_t)(rows ? rows[b] : b) * H;
  const bool any = d1 != nullptr || d2 != nullptr || e != nullptr || vec != nullptr;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float branches = 0.f;                          // the branches are summed first, then joined to the stream
    if (d1) branches = to_f32(d1[src + i]);
    if (d2) branches += to_f32(d2[src + i]);
    float v = resid[src + i] + branches;
    if (e) v += e[src + i];
    if (vec) v += vec[i];
    row[i] = v;
    if (any && !rows) resid[src + i] = v;
  }
  if (kind == NORM_NONE) return;
  __syncthreads();
  float mean, rstd;
  row_stats(row, H, kind, eps, part, mean, rstd);
  if (out_f32) {
    float* o = static_cast<float*>(out) + (size_t)b * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = (row[i] - mean) * rstd * (w ? w[i] : 1.f);
  } else {
    T* o = static_cast<T*>(out) + (size_t)b * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = from_f32<T>((row[i] - mean) * rstd * (w ? w[i] : 1.f));
  }
}

// dtype: the type of d1 and d2 (and of out unless out_f32).  Refuses rows wider than 51200.
KVB_EXPORT int kvb_join_norm(float* resid, const void* d1, const void* d2, const float* e, const float* vec,
                             const float* w, int kind, float eps, void* out, int out_f32, const int* rows,
                             int n_out_rows, int H, int dtype, cudaStream_t stream) {
  if (n_out_rows <= 0) return 0;
  if (kind < 0 || kind > 2) return KVB_ERR_BAD_SIZE;
  const size_t smem = (size_t)H * sizeof(float);
  if (smem > 200 * 1024) return KVB_ERR_BAD_SIZE;
  KVB_DISPATCH_DTYPE(dtype, T, {
    if (smem > 48 * 1024) {
      cudaError_t err = cudaFuncSetAttribute(join_norm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (err != cudaSuccess) return (int)err;
    }
    kvb_launch(join_norm_kernel<T>, dim3(n_out_rows), dim3(kRowThreads), smem, stream, resid, (const T*)d1,
               (const T*)d2, e, vec, w, kind, eps, out, out_f32, rows, H);
  });
  return kvb_launch_result();
}
