// A feed-forward made of many small experts of which every token uses a few.
//
//   * route_kernel: the router.  A block per up to eight tokens: logits z = W_r h in float32 (W_r float32, h as
//     stored; or handed in by the caller, who made them with a product of float32 sums), scores s = softmax(z) over
//     all experts (or, score_fn 1, s = sigmoid(z) of each), the `top` experts with the largest s + correction
//     (ties go to the lower index), their weights s / (sum of the chosen s + 1e-20) * scale (or, without renorm,
//     s * scale).  It
//     leaves a dense table gate[t, e] (0 for an expert that was not chosen) and, for the last
//     `identity` experts, which have no matrices and hand their input on, the sum of their weights.
//   * expert_act_kernel: the experts' first products lie side by side in one row, [E * F | shared];
//     a[t, j] = relu(p[t, j])^2 * gate[t, j / F] for j < E * F, relu(p)^2 behind it (an expert that
//     every token uses).  One product with the experts' stacked second matrices then adds up the chosen
//     experts' outputs, weighted, in its float32 accumulator; what an unchosen expert adds is exactly 0.
//   * limited_act_kernel: experts with a gate and an up product each, both limited, and the token's weight on the
//     expert's input instead of its output (see there).
//   * row_axpy_kernel: y[t] += c[t] * x[t], the identity experts' share.
// Every sum is taken in an order that depends on the sizes only, so a token's result does not
// depend on its neighbours in the step.
#include "common.cuh"

#include <math_constants.h>

constexpr int kRouteWarps = 8;
constexpr int kRouteTokens = 8;        // tokens a block routes at most: a router row is fetched once for all of them

// A block takes `tb` consecutive tokens (1, 2, 4 or 8, as many as their inputs fit shared memory).  Logits: warp w
// takes the w-th slice of K for every expert (two experts at a time, every load of the slice requested before the
// first is used); its lanes walk the slice (lane l the columns l, l + 32, ...) and keep one sum per token and expert,
// the lanes' sums are added across the warp, and the warps' sums in the order of the warps.  A token's sums are
// therefore taken in an order that depends on K only.  Then warp w chooses for the tokens w, w + 8, ...
template <typename T>
__global__ void __launch_bounds__(kRouteWarps * 32)
route_kernel(const T* __restrict__ h, int ld_h, const float* __restrict__ w_router, const float* __restrict__ logits,
             int ld_logits, const float* __restrict__ correction, float* __restrict__ gate,
             float* __restrict__ identity_weight, int T_, int K, int E, int n_identity, int top, float scale, int score_fn,
             int renorm, int tb) {
  extern __shared__ float smem[];
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t0 = blockIdx.x * tb;
  const int n_tok = min(tb, T_ - t0);
  const int n_all = E + n_identity;
  float* s_all = smem;                                  // [tb][n_all] logits, then scores
  float* c_all = s_all + (size_t)tb * n_all;            // [tb][n_all] choice scores; -inf once chosen
  float* part_all = c_all + (size_t)tb * n_all;         // [kRouteWarps][tb][n_all] the warps' sums (not with logits)
  float* x = part_all + (size_t)kRouteWarps * tb * n_all;   // [tb][K] the tokens' inputs, float32 (not with logits)
  if (logits != nullptr) {
    for (int i = threadIdx.x; i < n_tok * n_all; i += blockDim.x) {
      const int tt = i / n_all, e = i - tt * n_all;
      s_all[i] = logits[(size_t)(t0 + tt) * ld_logits + e];
    }
  } else {
    for (int i = threadIdx.x; i < n_tok * K; i += blockDim.x) {
      const int tt = i / K, k = i - tt * K;
      x[i] = to_f32(h[(size_t)(t0 + tt) * ld_h + k]);
    }
    for (int i = threadIdx.x + n_tok * K; i < tb * K; i += blockDim.x) x[i] = 0.f;
    __syncthreads();
    const int slice = ((K + kRouteWarps - 1) / kRouteWarps + 31) / 32 * 32;
    const int k0 = warp * slice, k1 = min(K, k0 + slice);
    for (int e0 = 0; e0 < n_all; e0 += 2) {
      const bool two = e0 + 1 < n_all;
      const float* wr0 = w_router + (size_t)e0 * K;
      const float* wr1 = w_router + (size_t)(two ? e0 + 1 : e0) * K;
      float p0[kRouteTokens], p1[kRouteTokens];
#pragma unroll
      for (int tt = 0; tt < kRouteTokens; ++tt) { p0[tt] = 0.f; p1[tt] = 0.f; }
#pragma unroll 8
      for (int k = k0 + lane; k < k1; k += 32) {
        const float a = wr0[k], b = wr1[k];
#pragma unroll
        for (int tt = 0; tt < kRouteTokens; ++tt) {
          if (tt < tb) {
            const float xv = x[tt * K + k];
            p0[tt] = fmaf(a, xv, p0[tt]);
            p1[tt] = fmaf(b, xv, p1[tt]);
          }
        }
      }
#pragma unroll
      for (int tt = 0; tt < kRouteTokens; ++tt) {
        if (tt >= tb) break;
        const float z0 = warp_sum(p0[tt]), z1 = warp_sum(p1[tt]);
        if (lane == 0) {
          part_all[((size_t)warp * tb + tt) * n_all + e0] = z0;
          if (two) part_all[((size_t)warp * tb + tt) * n_all + e0 + 1] = z1;
        }
      }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < tb * n_all; i += blockDim.x) {
      float z = 0.f;
      for (int w = 0; w < kRouteWarps; ++w) z += part_all[(size_t)w * tb * n_all + i];
      s_all[i] = z;
    }
  }
  __syncthreads();
  for (int tt = warp; tt < n_tok; tt += kRouteWarps) {
    const int t = t0 + tt;
    float* s = s_all + (size_t)tt * n_all;
    float* c = c_all + (size_t)tt * n_all;
    float sum = 1.f;
    if (score_fn == 0) {
      float zmax = -CUDART_INF_F;
      for (int e = lane; e < n_all; e += 32) zmax = fmaxf(zmax, s[e]);
      zmax = warp_max(zmax);
      sum = 0.f;
      for (int e = lane; e < n_all; e += 32) {
        const float v = expf(s[e] - zmax);
        s[e] = v;
        sum += v;
      }
      sum = warp_sum(sum);
    } else {
      for (int e = lane; e < n_all; e += 32) s[e] = 1.0f / (1.0f + expf(-s[e]));
    }
    __syncwarp();
    for (int e = lane; e < n_all; e += 32) {
      s[e] = s[e] / sum;
      c[e] = s[e] + (correction != nullptr ? correction[e] : 0.f);
      gate[(size_t)t * n_all + e] = 0.f;
    }
    __syncwarp();
    // the chosen experts, one after the other; their indices end up in lane 0 .. top - 1's `mine`
    int mine = -1;
    float chosen_sum = 0.f;
    for (int r = 0; r < top; ++r) {
      float best = -CUDART_INF_F;
      int at = 0x7fffffff;
      for (int e = lane; e < n_all; e += 32)
        if (c[e] > best) { best = c[e]; at = e; }       // ascending e: the lowest index among equals
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, at, o);
        if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
      }
      if (at == 0x7fffffff) break;                      // fewer experts than `top`
      if (lane == r) mine = at;
      chosen_sum += s[at];
      __syncwarp();
      if (lane == 0) c[at] = -CUDART_INF_F;
      __syncwarp();
    }
    const float norm = renorm ? scale / (chosen_sum + 1e-20f) : scale;
    float idw = 0.f;
    for (int r = 0; r < top; ++r) {
      const int e = __shfl_sync(0xffffffffu, mine, r);
      if (e < 0) continue;
      const float g = s[e] * norm;
      if (lane == 0) gate[(size_t)t * n_all + e] = g;
      if (e >= E) idw += g;
    }
    if (lane == 0 && identity_weight) identity_weight[t] = idw;
  }
}

// logits: float32 [T, >= E + n_identity] with row stride ld_logits, the router's products if the caller has made them
// (h and w_router are not read then), else null.  correction: may be null.  score_fn 0: softmax over all experts, 1: a
// sigmoid of each.  renorm 0: the chosen scores are the weights as they are (times scale).
// Refuses: more than 32 chosen experts per token, more than 4096 experts, K above 16384.
KVB_EXPORT int kvb_route(const void* h, int ld_h, const float* w_router, const float* logits, int ld_logits,
                         const float* correction, float* gate, float* identity_weight, int T_, int K, int E,
                         int n_identity, int top, float scale, int score_fn, int renorm, int dtype, cudaStream_t stream) {
  if (T_ <= 0) return 0;
  if (score_fn < 0 || score_fn > 1 || (logits != nullptr && ld_logits < E + n_identity)) return KVB_ERR_BAD_SIZE;
  if (E < 0 || n_identity < 0 || E + n_identity < 1 || E + n_identity > 4096 || top < 1 || top > 32 || K < 1 || K > 16384)
    return KVB_ERR_BAD_SIZE;
  const int n_all = E + n_identity;
  // as many tokens a block as their inputs fit 160 KB with, 8 at most; few tokens are spread over more blocks
  int tb = kRouteTokens;
  const size_t x_floats = logits ? 0 : (size_t)K + (size_t)kRouteWarps * n_all;
  // half of that once the step has blocks enough to fill the GPU either way: more blocks per SM hide more latency
  while (tb > 1 && ((size_t)tb * (x_floats + 2 * n_all) * sizeof(float) > 160 * 1024 || (T_ + tb - 1) / tb < 64)) tb >>= 1;
  if (tb == kRouteTokens && T_ / (tb / 2) >= 4 * kvb_sm_count()) tb >>= 1;
  const size_t smem = (size_t)tb * (x_floats + 2 * n_all) * sizeof(float);
  if (smem > 200 * 1024) return KVB_ERR_BAD_SIZE;
  KVB_DISPATCH_DTYPE(dtype, T, {
    if (smem > 48 * 1024) {
      cudaError_t err = cudaFuncSetAttribute(route_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (err != cudaSuccess) return (int)err;
    }
    kvb_launch(route_kernel<T>, dim3((T_ + tb - 1) / tb), dim3(kRouteWarps * 32), smem, stream, (const T*)h, ld_h, w_router,
               logits, ld_logits, correction, gate, identity_weight, T_, K, E, n_identity, top, scale, score_fn, renorm, tb);
  });
  return kvb_launch_result();
}

// p [T, E * F + S]: the first products of the E routed experts (F features each) and of one expert that
// every token uses (S features, may be 0).  gate [T, ld_gate] float32.  out [T, E * F + S] dense.
template <typename T>
__global__ void expert_act_kernel(const T* __restrict__ p, const float* __restrict__ gate, int ld_gate,
                                  T* __restrict__ out, int EF, int F, int width, size_t total) {
  pdl_trigger();
  pdl_wait();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / width;
    const int j = (int)(idx - t * width);
    const float g = j < EF ? gate[t * ld_gate + j / F] : 1.f;
    float a = 0.f;
    if (g != 0.f) {
      const float z = fmaxf(to_f32(p[idx]), 0.f);
      a = z * z * g;
    }
    out[idx] = from_f32<T>(a);
  }
}

// bfloat16 rows whose experts are multiples of 8 features wide: eight elements per thread, 16-byte accesses, one
// look at the token's weight for the expert.
__global__ void expert_act_bf16x8_kernel(const __nv_bfloat16* __restrict__ p, const float* __restrict__ gate, int ld_gate,
                                         __nv_bfloat16* __restrict__ out, int EF, int F, int width, size_t groups) {
  pdl_trigger();
  pdl_wait();
  const int gpr = width >> 3;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < groups;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / gpr;
    const int j = (int)(idx - t * gpr) << 3;
    const float g = j < EF ? gate[t * ld_gate + j / F] : 1.f;
    uint4 o = make_uint4(0u, 0u, 0u, 0u);
    if (g != 0.f) {
      const uint4 u = *reinterpret_cast<const uint4*>(p + t * width + j);
      const unsigned w[4] = {u.x, u.y, u.z, u.w};
      unsigned r[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float a = fmaxf(__uint_as_float(w[k] << 16), 0.f), b = fmaxf(__uint_as_float(w[k] & 0xffff0000u), 0.f);
        __nv_bfloat162 v = __floats2bfloat162_rn(a * a * g, b * b * g);
        r[k] = *reinterpret_cast<unsigned*>(&v);
      }
      o = make_uint4(r[0], r[1], r[2], r[3]);
    }
    *reinterpret_cast<uint4*>(out + t * width + j) = o;
  }
}

KVB_EXPORT int kvb_expert_act(const void* p, const float* gate, int ld_gate, void* out, int T_, int E, int F, int S,
                              int dtype, cudaStream_t stream) {
  if (T_ <= 0) return 0;
  const int width = E * F + S;
  if (E < 0 || F < 1 || S < 0 || width < 1) return KVB_ERR_BAD_SIZE;
  if (dtype == KVB_BF16 && F % 8 == 0 && S % 8 == 0 && (reinterpret_cast<uintptr_t>(p) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
    const size_t groups = (size_t)T_ * (width / 8);
    const size_t want8 = (groups + 255) / 256;
    const int blocks8 = (int)(want8 < (size_t)kvb_sm_count() * 16 ? want8 : (size_t)kvb_sm_count() * 16);
    kvb_launch(expert_act_bf16x8_kernel, dim3(blocks8), dim3(256), 0, stream, (const __nv_bfloat16*)p, gate, ld_gate,
               (__nv_bfloat16*)out, E * F, F, width, groups);
    return kvb_launch_result();
  }
  const size_t total = (size_t)T_ * width;
  const size_t want = (total + 255) / 256;
  const int blocks = (int)(want < (size_t)kvb_sm_count() * 16 ? want : (size_t)kvb_sm_count() * 16);
  KVB_DISPATCH_DTYPE(dtype, T, (kvb_launch(expert_act_kernel<T>, dim3(blocks), dim3(256), 0, stream, (const T*)p, gate,
                                            ld_gate, (T*)out, E * F, F, width, total)));
  return kvb_launch_result();
}

// Experts of the form  down (a(g) (u + 1)),  g = min(w gate.h, limit),  u = clamp(w up.h, -limit, limit),
// a(g) = g sigmoid(alpha g),  where w is the token's weight for the expert: it multiplies the expert's input, which for
// matrices without biases is the same as multiplying both first products, before the limits.
// p [T, ld_p]: per routed expert e its gate product (F features from column 2 e F) and its up product (the next F);
// behind the E routed experts one that every token uses: S gate features, then S up features, with a limit of its own
// and w = 1, whose result is multiplied by sigmoid(shared_logit[t * ld_s]) (float32; null: by 1), which for a last
// matrix without bias is the same as multiplying its output.  gate [T, ld_gate] float32: the weights, 0 for an expert
// that was not chosen.  out [T, E F + S + pad] dense, the padding columns zero.
template <typename T>
__global__ void limited_act_kernel(const T* __restrict__ p, int ld_p, const float* __restrict__ gate, int ld_gate,
                                   const float* __restrict__ shared_logit, int ld_s, T* __restrict__ out, int E, int F,
                                   int S, int width, float limit, float shared_limit, float alpha, size_t total) {
  pdl_trigger();
  pdl_wait();
  const int EF = E * F;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / width;
    const int j = (int)(idx - t * width);
    float a = 0.f;
    if (j < EF) {
      const int e = j / F, i = j - e * F;
      const float w = gate[t * ld_gate + e];
      if (w != 0.f) {
        const float g = fminf(w * to_f32(p[t * ld_p + 2 * e * F + i]), limit);
        const float u = fminf(fmaxf(w * to_f32(p[t * ld_p + 2 * e * F + F + i]), -limit), limit);
        a = g / (1.0f + expf(-alpha * g)) * (u + 1.0f);
      }
    } else if (j < EF + S) {
      const int i = j - EF;
      const float g = fminf(to_f32(p[t * ld_p + 2 * EF + i]), shared_limit);
      const float u = fminf(fmaxf(to_f32(p[t * ld_p + 2 * EF + S + i]), -shared_limit), shared_limit);
      a = g / (1.0f + expf(-alpha * g)) * (u + 1.0f);
      if (shared_logit != nullptr) a *= 1.0f / (1.0f + expf(-shared_logit[t * ld_s]));
    }
    out[idx] = from_f32<T>(a);
  }
}

// bfloat16 rows whose experts are multiples of 8 features wide: eight results per thread from two 16-byte loads, one
// look at the token's weight for the expert, and no load at all for an expert that was not chosen.
__device__ __forceinline__ float limited_one(float g, float u, float w, float limit, float alpha) {
  g = fminf(w * g, limit);
  u = fminf(fmaxf(w * u, -limit), limit);
  return g / (1.0f + expf(-alpha * g)) * (u + 1.0f);
}

__global__ void limited_act_bf16x8_kernel(const __nv_bfloat16* __restrict__ p, int ld_p, const float* __restrict__ gate,
                                          int ld_gate, const float* __restrict__ shared_logit, int ld_s,
                                          __nv_bfloat16* __restrict__ out, int E, int F, int S, int width, float limit,
                                          float shared_limit, float alpha, size_t groups) {
  pdl_trigger();
  pdl_wait();
  const int EF = E * F, gpr = width >> 3;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < groups;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / gpr;
    const int j = (int)(idx - t * gpr) << 3;
    uint4 o = make_uint4(0u, 0u, 0u, 0u);
    const __nv_bfloat16* gp = nullptr;
    const __nv_bfloat16* up = nullptr;
    float w = 0.f, lim = limit, post = 1.f;
    if (j < EF) {
      const int e = j / F, i = j - e * F;
      w = gate[t * ld_gate + e];
      gp = p + t * ld_p + 2 * e * F + i;
      up = gp + F;
    } else if (j < EF + S) {
      w = 1.f;
      lim = shared_limit;
      gp = p + t * ld_p + 2 * EF + (j - EF);
      up = gp + S;
      if (shared_logit != nullptr) post = 1.0f / (1.0f + expf(-shared_logit[t * ld_s]));
    }
    if (w != 0.f) {
      const uint4 g4 = *reinterpret_cast<const uint4*>(gp);
      const uint4 u4 = *reinterpret_cast<const uint4*>(up);
      const unsigned gw[4] = {g4.x, g4.y, g4.z, g4.w}, uw[4] = {u4.x, u4.y, u4.z, u4.w};
      unsigned r[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float a = limited_one(__uint_as_float(gw[k] << 16), __uint_as_float(uw[k] << 16), w, lim, alpha) * post;
        const float b = limited_one(__uint_as_float(gw[k] & 0xffff0000u), __uint_as_float(uw[k] & 0xffff0000u), w, lim,
                                    alpha) * post;
        __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
        r[k] = *reinterpret_cast<unsigned*>(&v);
      }
      o = make_uint4(r[0], r[1], r[2], r[3]);
    }
    *reinterpret_cast<uint4*>(out + t * width + j) = o;
  }
}

KVB_EXPORT int kvb_limited_act(const void* p, int ld_p, const float* gate, int ld_gate, const float* shared_logit,
                               int ld_s, void* out, int T_, int E, int F, int S, int pad, float limit, float shared_limit,
                               float alpha, int dtype, cudaStream_t stream) {
  if (T_ <= 0) return 0;
  const int width = E * F + S + pad;
  if (E < 0 || F < 1 || S < 0 || pad < 0 || E * F + S < 1 || ld_p < 2 * (E * F + S)) return KVB_ERR_BAD_SIZE;
  if (dtype == KVB_BF16 && F % 8 == 0 && S % 8 == 0 && pad % 8 == 0 && ld_p % 8 == 0 &&
      (reinterpret_cast<uintptr_t>(p) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
    const size_t groups = (size_t)T_ * (width / 8);
    const size_t want8 = (groups + 255) / 256;
    const int blocks8 = (int)(want8 < (size_t)kvb_sm_count() * 16 ? want8 : (size_t)kvb_sm_count() * 16);
    kvb_launch(limited_act_bf16x8_kernel, dim3(blocks8), dim3(256), 0, stream, (const __nv_bfloat16*)p, ld_p, gate, ld_gate,
               shared_logit, ld_s, (__nv_bfloat16*)out, E, F, S, width, limit, shared_limit, alpha, groups);
    return kvb_launch_result();
  }
  const size_t total = (size_t)T_ * width;
  const size_t want = (total + 255) / 256;
  const int blocks = (int)(want < (size_t)kvb_sm_count() * 16 ? want : (size_t)kvb_sm_count() * 16);
  KVB_DISPATCH_DTYPE(dtype, T, (kvb_launch(limited_act_kernel<T>, dim3(blocks), dim3(256), 0, stream, (const T*)p, ld_p,
                                            gate, ld_gate, shared_logit, ld_s, (T*)out, E, F, S, width, limit,
                                            shared_limit, alpha, total)));
  return kvb_launch_result();
}

// y[t, :] += c[t] * x[t, :]   (y [T, H] dense, x [T, >= H] with row stride ld_x)
template <typename T>
__global__ void row_axpy_kernel(T* __restrict__ y, const T* __restrict__ x, int ld_x, const float* __restrict__ c, int H,
                                size_t total) {
  pdl_trigger();
  pdl_wait();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / H;
    const int i = (int)(idx - t * H);
    const float w = c[t];
    if (w != 0.f) y[idx] = from_f32<T>(fmaf(w, to_f32(x[t * ld_x + i]), to_f32(y[idx])));
  }
}

KVB_EXPORT int kvb_row_axpy(void* y, const void* x, int ld_x, const float* c, int T_, int H, int dtype,
                            cudaStream_t stream) {
  if (T_ <= 0 || H <= 0) return 0;
  const size_t total = (size_t)T_ * H;
  const size_t want = (total + 255) / 256;
  const int blocks = (int)(want < (size_t)kvb_sm_count() * 16 ? want : (size_t)kvb_sm_count() * 16);
  KVB_DISPATCH_DTYPE(dtype, T, (kvb_launch(row_axpy_kernel<T>, dim3(blocks), dim3(256), 0, stream, (T*)y, (const T*)x,
                                            ld_x, c, H, total)));
  return kvb_launch_result();
}
