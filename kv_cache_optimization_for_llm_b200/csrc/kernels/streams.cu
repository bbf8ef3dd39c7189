// A residual stream kept as several copies ("streams") that every sublayer reads as a weighted sum
// and writes back through a small mixing matrix, the token shift in front of a mixer, the
// sinusoidal position vector added to the embedding, and the xIELU activation.
//
//   embed_sinusoid_streams   x = table[token] + sinusoid(position), copied into every stream
//   hyper_norm               the pending write of the sublayer before (x_t <- sum_s mix[s, t] x_s + out[t] y),
//                            the read of the next one (u = sum_s in[s] x_s) and its RMS norm, one launch;
//                            for steps of single tokens also the token shift behind the norm
//   token_shift              h <- h + (h_prev - h) * shift along each request's tokens, the last normed
//                            row of a request kept in its state slot
//   xielu                    the activation of the dense feed-forward
//
// Everything here is float32 arithmetic on a float32 stream; only branch outputs and the normed rows
// handed to the products have the compute type.  With one stream, in = mix = out = 1 this is the
// ordinary residual add in front of a norm.
#include "common.cuh"

#include <math_constants.h>

constexpr int kMaxStreams = 8;

__device__ __forceinline__ float block_sum_f(float v, float* part) {
  v = warp_sum(v);
  __syncthreads();                       // part may still be read from the call before
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
  const int nw = blockDim.x >> 5;
  for (int i = 0; i < nw; ++i) t += part[i];      // the same order in every thread
  return t;
}

// ---------------------------------------------------------------- embedding + position vector
// Entry 2i of the position vector is sin(p f_i), entry 2i + 1 is cos(p f_i), f_i = base^(-2i / W).  The angle is
// formed in double precision (positions times a frequency lose bits in float32 beyond a few thousand).
template <typename T>
__global__ void embed_sinusoid_streams_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                              const int* __restrict__ sampled, int n_sampled,
                                              const int* __restrict__ positions, float* __restrict__ x, int S, int W,
                                              int V, float base, int* status) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 && sampled && -(id + 1) < n_sampled) id = sampled[-(id + 1)];
  const bool bad = id < 0 || id >= V;
  if (bad && threadIdx.x == 0) atomicCAS(status, 0, KVB_STATUS_BAD_TOKEN);
  const T* row = table + (size_t)(bad ? 0 : id) * W;
  const double p = (double)positions[t];
  const double lb = log((double)base);
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    const int i = c >> 1;
    const double angle = p * exp(-(2.0 * i / (double)W) * lb);
    const float pe = (float)((c & 1) ? cos(angle) : sin(angle));
    const float v = bad ? 0.f : to_f32(row[c]) + pe;
    for (int s = 0; s < S; ++s) x[((size_t)t * S + s) * W + c] = v;
  }
}

KVB_EXPORT int kvb_embed_sinusoid_streams(const void* table, int dtype, const int* ids, const int* sampled,
                                          int n_sampled, const int* positions, float* x, int T_, int S, int W, int V,
                                          float base, int* status, cudaStream_t stream) {
  if (T_ <= 0) return 0;
  if (S < 1 || S > kMaxStreams || W < 1) return KVB_ERR_BAD_SIZE;
  KVB_DISPATCH_DTYPE(dtype, T, (kvb_launch(embed_sinusoid_streams_kernel<T>, dim3(T_), dim3(W >= 1024 ? 256 : 128), 0,
                                            stream, (const T*)table, ids, sampled, n_sampled, positions, x, S, W, V, base,
                                            status)));
  return kvb_launch_result();
}

// ---------------------------------------------------------------- streams: write, read, norm (and shift)
struct HyperArgs {
  float* x;               // [T, S, W] the streams
  const void* y;          // [T, W] compute type: the pending sublayer output, or null
  const void* y2;         // a second output that joins the first (two mixers side by side), or null
  const float* mix;       // [S, S] indexed [from, to], or null (identity)
  const float* out_w;     // [S] or null (ones)
  const float* in_w;      // [S] or null (ones: the plain sum of the streams)
  const float* weight;    // [W] or null
  const int* rows;        // null, or the rows to produce (the streams are then left as they are)
  void* out;              // [n, W], or null (only the write is carried out)
  int n, S, W;
  float eps;
  int one_plus;           // the norm multiplies by 1 + weight
  int out_f32;            // out is float32 whatever the compute type
  // the token shift behind the norm, for steps in which every request brings one token
  const float* shift;     // [W] or null
  float* shift_state;     // the last normed row of slot 0, slot_stride floats from slot to slot
  long long slot_stride;
  const int* slots;       // [n]
  const int* positions;   // [n]
  // for steps with runs of tokens: where the first token of each run finds the row before it
  float* prev;            // [R, W] or null
  const int* token_req;   // [T]
  const int* q_start;     // [R + 1]
};

template <typename T>
__global__ void __launch_bounds__(256) hyper_norm_kernel(HyperArgs a) {
  extern __shared__ float hs[];
  float* u_s = hs;                               // [W]
  __shared__ float part[8];
  __shared__ float mix_s[kMaxStreams * kMaxStreams], out_s[kMaxStreams], in_s[kMaxStreams];
  pdl_trigger();
  const int S = a.S, W = a.W;
  for (int i = threadIdx.x; i < S * S; i += blockDim.x)
    mix_s[i] = a.mix ? a.mix[i] : ((i / S == i % S) ? 1.f : 0.f);
  for (int i = threadIdx.x; i < S; i += blockDim.x) {
    out_s[i] = a.out_w ? a.out_w[i] : 1.f;
    in_s[i] = a.in_w ? a.in_w[i] : 1.f;
  }
  pdl_wait();
  __syncthreads();
  const int b = blockIdx.x;
  const int t = a.rows ? a.rows[b] : b;
  float* xt = a.x + (size_t)t * S * W;
  const T* y = a.y ? static_cast<const T*>(a.y) + (size_t)t * W : nullptr;
  const T* y2 = a.y2 ? static_cast<const T*>(a.y2) + (size_t)t * W : nullptr;
  const bool store = a.rows == nullptr && y != nullptr;
  float sq = 0.f;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float old[kMaxStreams];
#pragma unroll
    for (int s = 0; s < kMaxStreams; ++s) old[s] = s < S ? xt[(size_t)s * W + c] : 0.f;
    float u = 0.f;
    if (y != nullptr) {
      const float yv = to_f32(y[c]) + (y2 != nullptr ? to_f32(y2[c]) : 0.f);
#pragma unroll
      for (int r = 0; r < kMaxStreams; ++r) {
        if (r >= S) break;
        float v = out_s[r] * yv;
#pragma unroll
        for (int s = 0; s < kMaxStreams; ++s)
          if (s < S) v = fmaf(mix_s[s * S + r], old[s], v);
        if (store) xt[(size_t)r * W + c] = v;
        u = fmaf(in_s[r], v, u);
      }
    } else {
#pragma unroll
      for (int s = 0; s < kMaxStreams; ++s)
        if (s < S) u = fmaf(in_s[s], old[s], u);
    }
    u_s[c] = u;
    sq = fmaf(u, u, sq);
  }
  if (a.out == nullptr) return;
  const float total = block_sum_f(sq, part);
  const float rstd = 1.0f / sqrtf(total / (float)W + a.eps);
  const bool first_of_run = a.prev != nullptr && a.q_start[a.token_req[t]] == t;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float h = u_s[c] * rstd;
    if (a.weight) h *= a.one_plus ? 1.0f + a.weight[c] : a.weight[c];
    if (a.shift != nullptr) {
      float* st = a.shift_state + (size_t)a.slots[b] * a.slot_stride;
      const float before = a.positions[b] > 0 ? st[c] : 0.f;
      st[c] = h;
      h = fmaf(before - h, a.shift[c], h);
    } else if (first_of_run) {
      // the row in front of this run's first token: from the request's slot, zero at the sequence's start
      const int r = a.token_req[t];
      const float* st = a.shift_state + (size_t)a.slots[r] * a.slot_stride;
      a.prev[(size_t)r * W + c] = a.positions[t] > 0 ? st[c] : 0.f;
    }
    if (a.out_f32) static_cast<float*>(a.out)[(size_t)b * W + c] = h;
    else static_cast<T*>(a.out)[(size_t)b * W + c] = from_f32<T>(h);
  }
}

KVB_EXPORT int kvb_hyper_norm(const HyperArgs* args, int dtype, cudaStream_t stream) {
  HyperArgs a = *args;
  if (a.n <= 0) return 0;
  if (a.S < 1 || a.S > kMaxStreams || a.W < 1 || (size_t)a.W * sizeof(float) > 160 * 1024) return KVB_ERR_BAD_SIZE;
  const size_t smem = (size_t)a.W * sizeof(float);
  KVB_DISPATCH_DTYPE(dtype, T, {
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(hyper_norm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
    }
    kvb_launch(hyper_norm_kernel<T>, dim3(a.n), dim3(a.W >= 1024 ? 256 : 128), smem, stream, a);
  });
  return kvb_launch_result();
}

// ---------------------------------------------------------------- token shift over runs of tokens
// h [T, W] float32: the normed rows.  out[t] = h[t] + (before - h[t]) * shift, before = h[t - 1] inside a run and
// prev[request] for the run's first token.  The run's last row goes to the request's slot.
template <typename T>
__global__ void token_shift_kernel(const float* __restrict__ h, const float* __restrict__ prev,
                                   const float* __restrict__ shift, float* __restrict__ state, long long slot_stride,
                                   const int* __restrict__ slots, const int* __restrict__ token_req,
                                   const int* __restrict__ q_start, T* __restrict__ out, int W) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int r = token_req[t];
  const bool first = q_start[r] == t, last = q_start[r + 1] == t + 1;
  const float* before = first ? prev + (size_t)r * W : h + (size_t)(t - 1) * W;
  float* st = state + (size_t)slots[r] * slot_stride;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    const float v = h[(size_t)t * W + c];
    out[(size_t)t * W + c] = from_f32<T>(fmaf(before[c] - v, shift[c], v));
    if (last) st[c] = v;
  }
}

KVB_EXPORT int kvb_token_shift(const float* h, const float* prev, const float* shift, float* state,
                               long long slot_stride, const int* slots, const int* token_req, const int* q_start,
                               void* out, int T_, int W, int dtype, cudaStream_t stream) {
  if (T_ <= 0) return 0;
  if (W < 1) return KVB_ERR_BAD_SIZE;
  KVB_DISPATCH_DTYPE(dtype, T, (kvb_launch(token_shift_kernel<T>, dim3(T_), dim3(W >= 1024 ? 256 : 128), 0, stream, h,
                                            prev, shift, state, slot_stride, slots, token_req, q_start, (T*)out, W)));
  return kvb_launch_result();
}

// ---------------------------------------------------------------- xIELU
// z > 0: ap z^2 + z / 2;  z <= 0: an (exp(z) - 1 - z) + z / 2, with ap = softplus(p), an = 1/2 + softplus(q),
// p and q the two numbers of `pq`.
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

__device__ __forceinline__ float xielu_f(float z, float ap, float an) {
  return z > 0.f ? fmaf(ap * z, z, 0.5f * z) : fmaf(an, expm1f(z) - z, 0.5f * z);
}

template <typename T>
__global__ void xielu_kernel(const T* __restrict__ in, T* __restrict__ out, long long n, const float* __restrict__ pq) {
  pdl_trigger();
  const float ap = softplus_f(pq[0]), an = 0.5f + softplus_f(pq[1]);
  pdl_wait();
  const long long i0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i0 >= n) return;
  if (i0 + 8 <= n && sizeof(T) == 2) {
    const uint4 u = *reinterpret_cast<const uint4*>(in + i0);
    const unsigned w[4] = {u.x, u.y, u.z, u.w};
    unsigned o[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float lo = xielu_f(__uint_as_float(w[e] << 16), ap, an);
      const float hi = xielu_f(__uint_as_float(w[e] & 0xffff0000u), ap, an);
      __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
      o[e] = *reinterpret_cast<unsigned*>(&v);
    }
    *reinterpret_cast<uint4*>(out + i0) = make_uint4(o[0], o[1], o[2], o[3]);
    return;
  }
  for (long long i = i0; i < n && i < i0 + 8; ++i) out[i] = from_f32<T>(xielu_f(to_f32(in[i]), ap, an));
}

KVB_EXPORT int kvb_xielu(const void* in, void* out, long long n, const float* pq, int dtype, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (((uintptr_t)in % 16) || ((uintptr_t)out % 16)) return KVB_ERR_ALIGN;
  const long long units = (n + 7) / 8;
  KVB_DISPATCH_DTYPE(dtype, T, (kvb_launch(xielu_kernel<T>, dim3((unsigned)((units + 255) / 256)), dim3(256), 0, stream,
                                            (const T*)in, (T*)out, n, pq)));
  return kvb_launch_result();
}
