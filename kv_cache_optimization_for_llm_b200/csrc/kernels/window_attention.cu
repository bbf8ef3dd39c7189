// Attention over a paged cache whose rows hold a token's key and value side by side, for
// mixers that differ from the rotary kind in their mask and their softmax:
//   * key and value sizes of their own (Dk, Dv); a cached row is [k (Dk) | v (Dv)] per token and
//     key/value head, the pool being [pages, kv heads, page size, Dk + Dv];
//   * a sliding window that also keeps the sequence's first tokens: query i sees key j when
//     j <= i and (i - j < window or j < keep_first); window 0: every key up to i;
//   * a softmax whose denominator may count one more (a key of score 0 that has no value):
//     p_j = exp(s_j) / (1 + sum exp(s_j)).
// Positions do not enter the scores here; a mixer that rotates does so before it calls.
//
// window_attention_kernel: one block per (query token, query head), any mix of runs and single
// tokens; its four warps take the keys in chunks of 32 consecutive positions, chunk c going to
// warp c % 4, so the sums a query sees follow absolute positions and do not depend on how its
// request was cut into steps, on the batch or on where the pages lie.  Everything is float32
// but the cached rows and the query as they are stored.
#include "common.cuh"
#include "score_shape.cuh"

#include <math_constants.h>

constexpr int kMaxDim = 256;
constexpr int kWarps = 4;

// Writes the step's keys and values into their requests' pages.  src [T, >= ...] holds, per token, the
// keys of all kv heads from column k_off on (G * Dk) and the values from v_off on (G * Dv).
template <typename T>
__global__ void kv_rows_append_kernel(const T* __restrict__ src, int ld, int k_off, int v_off, T* __restrict__ pages,
                                      const int* __restrict__ block_table, int max_pages, int page_size, int num_pages,
                                      const int* __restrict__ positions, const int* __restrict__ token_req, int G,
                                      int Dk, int Dv, int* status) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, g = blockIdx.y;
  const int pos = positions[t];
  const int lp = pos / page_size;
  const int page = lp < max_pages ? block_table[(size_t)token_req[t] * max_pages + lp] : -1;
  if (page < 0 || page >= num_pages) {
    if (threadIdx.x == 0) atomicCAS(status, 0, KVB_STATUS_UNMAPPED_PAGE);
    return;
  }
  T* row = pages + (((size_t)page * G + g) * page_size + (pos % page_size)) * (Dk + Dv);
  const T* k = src + (size_t)t * ld + k_off + g * Dk;
  const T* v = src + (size_t)t * ld + v_off + g * Dv;
  for (int i = threadIdx.x; i < Dk; i += blockDim.x) row[i] = k[i];
  for (int i = threadIdx.x; i < Dv; i += blockDim.x) row[Dk + i] = v[i];
}

KVB_EXPORT int kvb_kv_rows_append(const void* src, int ld, int k_off, int v_off, void* pages, const int* block_table,
                                  int max_pages, int page_size, int num_pages, const int* positions,
                                  const int* token_req, int T_, int G, int Dk, int Dv, int dtype, int* status,
                                  cudaStream_t stream) {
  if (T_ <= 0) return 0;
  if (G < 1 || Dk < 1 || Dv < 1) return KVB_ERR_BAD_SIZE;
  KVB_DISPATCH_DTYPE(dtype, T, (kvb_launch(kv_rows_append_kernel<T>, dim3(T_, G), dim3(64), 0, stream, (const T*)src, ld,
                                            k_off, v_off, (T*)pages, block_table, max_pages, page_size, num_pages,
                                            positions, token_req, G, Dk, Dv, status)));
  return kvb_launch_result();
}

// The dot product of the query (float32, shared memory) with a cached key; 16-byte loads when
// the rows allow it.
template <typename T>
__device__ __forceinline__ float key_dot(const float* q_s, const T* k, int Dk, bool vec);

template <>
__device__ __forceinline__ float key_dot<float>(const float* q_s, const float* k, int Dk, bool vec) {
  float dot = 0.f;
  if (vec) {
    for (int i = 0; i < Dk; i += 4) {
      const float4 x = *reinterpret_cast<const float4*>(k + i);
      dot = fmaf(q_s[i], x.x, dot); dot = fmaf(q_s[i + 1], x.y, dot);
      dot = fmaf(q_s[i + 2], x.z, dot); dot = fmaf(q_s[i + 3], x.w, dot);
    }
  } else {
    for (int i = 0; i < Dk; ++i) dot = fmaf(q_s[i], k[i], dot);
  }
  return dot;
}

template <>
__device__ __forceinline__ float key_dot<__nv_bfloat16>(const float* q_s, const __nv_bfloat16* k, int Dk, bool vec) {
  float dot = 0.f;
  if (vec) {
    for (int i = 0; i < Dk; i += 8) {
      const uint4 x = *reinterpret_cast<const uint4*>(k + i);
      const unsigned w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        dot = fmaf(q_s[i + 2 * u], __uint_as_float(w[u] << 16), dot);
        dot = fmaf(q_s[i + 2 * u + 1], __uint_as_float(w[u] & 0xffff0000u), dot);
      }
    }
  } else {
    for (int i = 0; i < Dk; ++i) dot = fmaf(q_s[i], __bfloat162float(k[i]), dot);
  }
  return dot;
}

template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
window_attention_kernel(const T* __restrict__ q_base, int q_row_stride, const T* __restrict__ pages,
                        const int* __restrict__ block_table, int max_pages, int page_size, int num_pages,
                        const int* __restrict__ positions, const int* __restrict__ token_req, T* __restrict__ out,
                        int nq, int nkv, int Dk, int Dv, float scale, int window, int keep_first, int one_more,
                        int vec, ScoreShape shape, int* status) {
  __shared__ float q_s[kMaxDim];
  __shared__ float acc_s[kWarps][kMaxDim];
  __shared__ float m_s[kWarps], l_s[kWarps];

  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y;
  const int hk = h / (nq / nkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pos = positions[t];
  const int* table = block_table + (size_t)token_req[t] * max_pages;
  const int row_len = Dk + Dv;
  const int lo = first_seen_key(pos, window, shape.chunk);       // first key of the window or of the position's block
  const int keep = window > 0 ? keep_first : 0;                  // keys below it are seen whatever the window
  const int keep_chunks = (keep + 31) / 32;
  const int lo_chunk = lo / 32;

  const T* q = q_base + (size_t)t * q_row_stride + (size_t)h * Dk;
  for (int i = threadIdx.x; i < Dk; i += blockDim.x) q_s[i] = to_f32(q[i]);
  __syncthreads();

  float m = -CUDART_INF_F, l = 0.f;
  float acc[kMaxDim / 32];
#pragma unroll
  for (int r = 0; r < kMaxDim / 32; ++r) acc[r] = 0.f;

  for (int c = warp; c * 32 <= pos; c += kWarps) {
    if (c >= keep_chunks && c < lo_chunk) {
      // between the kept first tokens and the window: on to this warp's first chunk of the window
      c += (lo_chunk - c + kWarps - 1) / kWarps * kWarps - kWarps;
      continue;
    }
    const int j = c * 32 + lane;
    const bool valid = j <= pos && (j >= lo || j < keep);
    long long off = -1;
    float s = -CUDART_INF_F;
    if (valid) {
      const int lp = j / page_size;
      const int page = lp < max_pages ? table[lp] : -1;
      if (page < 0 || page >= num_pages) {
        atomicCAS(status, 0, KVB_STATUS_UNMAPPED_PAGE);
      } else {
        off = (((long long)page * nkv + hk) * page_size + (j % page_size)) * row_len;
        s = shape_score(key_dot<T>(q_s, pages + off, Dk, vec != 0) * scale, shape, h, pos - j);
      }
    }
    const float cm = warp_max(s);
    if (cm == -CUDART_INF_F) continue;
    const float m_new = fmaxf(m, cm);
    const float corr = (m == -CUDART_INF_F) ? 0.f : expf(m - m_new);
    const float p = (off >= 0) ? expf(s - m_new) : 0.f;
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int r = 0; r < kMaxDim / 32; ++r) acc[r] *= corr;
    const int n_in_chunk = min(32, pos - c * 32 + 1);
    for (int jj = 0; jj < n_in_chunk; ++jj) {
      const long long oj = __shfl_sync(0xffffffffu, off, jj);
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      if (oj < 0) continue;
      const T* v = pages + oj + Dk;
#pragma unroll
      for (int r = 0; r < kMaxDim / 32; ++r) {
        const int i = r * 32 + lane;
        if (i < Dv) acc[r] = fmaf(pj, to_f32(v[i]), acc[r]);
      }
    }
    m = m_new;
  }

  if (lane == 0) { m_s[warp] = m; l_s[warp] = l; }
#pragma unroll
  for (int r = 0; r < kMaxDim / 32; ++r) {
    const int i = r * 32 + lane;
    if (i < Dv) acc_s[warp][i] = acc[r];
  }
  __syncthreads();
  if (warp == 0) {
    // what joins the denominator without a value: a key of score 0, or the head's learned score
    const float extra = one_more ? 0.f : (shape.sinks != nullptr ? shape.sinks[h] : -CUDART_INF_F);
    float M = extra;
    for (int w = 0; w < kWarps; ++w) M = fmaxf(M, m_s[w]);
    float L = extra == -CUDART_INF_F ? 0.f : expf(extra - M), f[kWarps];
    for (int w = 0; w < kWarps; ++w) {
      f[w] = (m_s[w] == -CUDART_INF_F) ? 0.f : expf(m_s[w] - M);
      L += l_s[w] * f[w];
    }
    T* o = out + ((size_t)t * nq + h) * Dv;
    const T* gate = shape.gate ? static_cast<const T*>(shape.gate) + (size_t)t * shape.gate_ld + (size_t)h * Dv : nullptr;
    for (int i = lane; i < Dv; i += 32) {
      float a = 0.f;
      for (int w = 0; w < kWarps; ++w) a += acc_s[w][i] * f[w];
      a = L > 0.f ? a / L * shape.out_scale : 0.f;
      if (gate != nullptr) a *= 1.0f / (1.0f + expf(-to_f32(gate[i])));
      o[i] = from_f32<T>(a);
    }
  }
}

// The same attention with the query heads that share a key/value head in one block: a cached row is read
// once for all of them.  One block per (query token, key/value head); chunk c of 32 keys goes to warp
// c % kGroupWarps as above; a lane scores its key against every head of the group, and in the weighted sum
// owns VPL consecutive value channels (one vector load per key).  Takes groups of up to 8 heads and values
// of up to 128 channels that are a multiple of 32 wide; the launcher falls back to the kernel above otherwise.
constexpr int kGroupWarps = 8;
constexpr int kMaxGroup = 8;

template <typename T, int VPL>
__device__ __forceinline__ void load_values(const T* v, float* x);
template <> __device__ __forceinline__ void load_values<float, 1>(const float* v, float* x) { x[0] = v[0]; }
template <> __device__ __forceinline__ void load_values<float, 2>(const float* v, float* x) {
  const float2 a = *reinterpret_cast<const float2*>(v); x[0] = a.x; x[1] = a.y;
}
template <> __device__ __forceinline__ void load_values<float, 4>(const float* v, float* x) {
  const float4 a = *reinterpret_cast<const float4*>(v); x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
}
template <> __device__ __forceinline__ void load_values<__nv_bfloat16, 1>(const __nv_bfloat16* v, float* x) {
  x[0] = __bfloat162float(v[0]);
}
template <> __device__ __forceinline__ void load_values<__nv_bfloat16, 2>(const __nv_bfloat16* v, float* x) {
  const unsigned a = *reinterpret_cast<const unsigned*>(v);
  x[0] = __uint_as_float(a << 16); x[1] = __uint_as_float(a & 0xffff0000u);
}
template <> __device__ __forceinline__ void load_values<__nv_bfloat16, 4>(const __nv_bfloat16* v, float* x) {
  const uint2 a = *reinterpret_cast<const uint2*>(v);
  x[0] = __uint_as_float(a.x << 16); x[1] = __uint_as_float(a.x & 0xffff0000u);
  x[2] = __uint_as_float(a.y << 16); x[3] = __uint_as_float(a.y & 0xffff0000u);
}

__device__ __forceinline__ void load_16_bytes(const float* p, float* x) {
  const float4 u = *reinterpret_cast<const float4*>(p);
  x[0] = u.x; x[1] = u.y; x[2] = u.z; x[3] = u.w;
}
__device__ __forceinline__ void load_16_bytes(const __nv_bfloat16* p, float* x) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const unsigned w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int e = 0; e < 4; ++e) { x[2 * e] = __uint_as_float(w[e] << 16); x[2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u); }
}

// Small groups and values keep to 64 registers, so that four blocks share an SM (a decode step of 64 requests and
// 8 key/value heads is then one round of blocks, not one and a seventh).
template <typename T, int VPL, int GP>
__global__ void __launch_bounds__(kGroupWarps * 32, (GP * VPL <= 8) ? 4 : 1)
window_attention_group_kernel(const T* __restrict__ q_base, int q_row_stride, const T* __restrict__ pages,
                              const int* __restrict__ block_table, int max_pages, int page_size, int num_pages,
                              const int* __restrict__ positions, const int* __restrict__ token_req, T* __restrict__ out,
                              int nq, int nkv, int Dk, float scale, int window, int keep_first, int one_more, int vec,
                              ScoreShape shape, int* status) {
  constexpr int Dv = VPL * 32;
  extern __shared__ float gsm[];
  float* q_s = gsm;                                  // [GP][Dk]
  float* acc_s = q_s + GP * Dk;                      // [kGroupWarps][GP][Dv]
  float* m_s = acc_s + kGroupWarps * GP * Dv;        // [kGroupWarps][GP]
  float* l_s = m_s + kGroupWarps * GP;               // [kGroupWarps][GP]

  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, hk = blockIdx.y;
  const int G = nq / nkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pos = positions[t];
  const int* table = block_table + (size_t)token_req[t] * max_pages;
  const int row_len = Dk + Dv;
  const int lo = first_seen_key(pos, window, shape.chunk);
  const int keep = window > 0 ? keep_first : 0;
  const int keep_chunks = (keep + 31) / 32;
  const int lo_chunk = lo / 32;

  const T* q = q_base + (size_t)t * q_row_stride + (size_t)hk * G * Dk;
  for (int i = threadIdx.x; i < GP * Dk; i += blockDim.x) q_s[i] = (i < G * Dk) ? to_f32(q[i]) : 0.f;
  __syncthreads();

  float m[GP], l[GP], acc[GP][VPL];
#pragma unroll
  for (int g = 0; g < GP; ++g) {
    m[g] = -CUDART_INF_F; l[g] = 0.f;
#pragma unroll
    for (int r = 0; r < VPL; ++r) acc[g][r] = 0.f;
  }

  for (int c = warp; c * 32 <= pos; c += kGroupWarps) {
    if (c >= keep_chunks && c < lo_chunk) {
      c += (lo_chunk - c + kGroupWarps - 1) / kGroupWarps * kGroupWarps - kGroupWarps;
      continue;
    }
    const int j = c * 32 + lane;
    const bool valid = j <= pos && (j >= lo || j < keep);
    long long off = -1;
    float s[GP];
#pragma unroll
    for (int g = 0; g < GP; ++g) s[g] = -CUDART_INF_F;
    if (valid) {
      const int lp = j / page_size;
      const int page = lp < max_pages ? table[lp] : -1;
      if (page < 0 || page >= num_pages) {
        atomicCAS(status, 0, KVB_STATUS_UNMAPPED_PAGE);
      } else {
        off = (((long long)page * nkv + hk) * page_size + (j % page_size)) * row_len;
        const T* k = pages + off;
        float dot[GP];
#pragma unroll
        for (int g = 0; g < GP; ++g) dot[g] = 0.f;
        if (vec) {
          constexpr int PER = 16 / (int)sizeof(T);
#pragma unroll 4
          for (int i = 0; i < Dk; i += PER) {     // unrolled: the row's loads are all requested before the first is used
            float x[PER];
            load_16_bytes(k + i, x);
#pragma unroll
            for (int e4 = 0; e4 < PER; e4 += 4) {
#pragma unroll
              for (int g = 0; g < GP; ++g) {
                const float4 qv = *reinterpret_cast<const float4*>(q_s + g * Dk + i + e4);
                dot[g] = fmaf(qv.x, x[e4], dot[g]); dot[g] = fmaf(qv.y, x[e4 + 1], dot[g]);
                dot[g] = fmaf(qv.z, x[e4 + 2], dot[g]); dot[g] = fmaf(qv.w, x[e4 + 3], dot[g]);
              }
            }
          }
        } else {
          for (int i = 0; i < Dk; ++i) {
            const float x = to_f32(k[i]);
#pragma unroll
            for (int g = 0; g < GP; ++g) dot[g] = fmaf(q_s[g * Dk + i], x, dot[g]);
          }
        }
#pragma unroll
        for (int g = 0; g < GP; ++g) s[g] = g < G ? shape_score(dot[g] * scale, shape, hk * G + g, pos - j) : 0.f;
      }
    }
    if (warp_max(off >= 0 ? 1.f : -CUDART_INF_F) == -CUDART_INF_F) continue;   // nothing readable in this chunk
    float p[GP];
#pragma unroll
    for (int g = 0; g < GP; ++g) {
      const float m_new = fmaxf(m[g], warp_max(s[g]));
      const float corr = (m[g] == -CUDART_INF_F) ? 0.f : expf(m[g] - m_new);
      p[g] = (off >= 0) ? expf(s[g] - m_new) : 0.f;
      l[g] = l[g] * corr + warp_sum(p[g]);
#pragma unroll
      for (int r = 0; r < VPL; ++r) acc[g][r] *= corr;
      m[g] = m_new;
    }
    // the values of eight keys are requested together: one key's load after the other would cost a trip to memory each
    const int n_in_chunk = min(32, pos - c * 32 + 1);
    for (int jj0 = 0; jj0 < n_in_chunk; jj0 += 8) {
      float x[8][VPL];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const long long oj = __shfl_sync(0xffffffffu, off, (jj0 + u) & 31);
        if (oj >= 0 && jj0 + u < n_in_chunk) {
          load_values<T, VPL>(pages + oj + Dk + lane * VPL, x[u]);
        } else {
#pragma unroll
          for (int r = 0; r < VPL; ++r) x[u][r] = 0.f;
        }
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
#pragma unroll
        for (int g = 0; g < GP; ++g) {
          const float pj = __shfl_sync(0xffffffffu, p[g], (jj0 + u) & 31);     // 0 for a key that is not seen
#pragma unroll
          for (int r = 0; r < VPL; ++r) acc[g][r] = fmaf(pj, x[u][r], acc[g][r]);
        }
      }
    }
  }

#pragma unroll
  for (int g = 0; g < GP; ++g) {
    if (lane == 0) { m_s[warp * GP + g] = m[g]; l_s[warp * GP + g] = l[g]; }
#pragma unroll
    for (int r = 0; r < VPL; ++r) acc_s[(warp * GP + g) * Dv + lane * VPL + r] = acc[g][r];
  }
  __syncthreads();
  // warp g finishes head g: the warps' partial sums are merged in the order of the warps
  for (int g = warp; g < G; g += kGroupWarps) {
    const int hq = hk * G + g;
    const float extra = one_more ? 0.f : (shape.sinks != nullptr ? shape.sinks[hq] : -CUDART_INF_F);
    float M = extra;
    for (int w = 0; w < kGroupWarps; ++w) M = fmaxf(M, m_s[w * GP + g]);
    float L = extra == -CUDART_INF_F ? 0.f : expf(extra - M), f[kGroupWarps];
    for (int w = 0; w < kGroupWarps; ++w) {
      const float mw = m_s[w * GP + g];
      f[w] = (mw == -CUDART_INF_F) ? 0.f : expf(mw - M);
      L += l_s[w * GP + g] * f[w];
    }
    T* o = out + ((size_t)t * nq + hq) * Dv;
    const T* gate = shape.gate ? static_cast<const T*>(shape.gate) + (size_t)t * shape.gate_ld + (size_t)hq * Dv : nullptr;
    for (int i = lane; i < Dv; i += 32) {
      float a = 0.f;
      for (int w = 0; w < kGroupWarps; ++w) a += acc_s[(w * GP + g) * Dv + i] * f[w];
      a = L > 0.f ? a / L * shape.out_scale : 0.f;
      if (gate != nullptr) a *= 1.0f / (1.0f + expf(-to_f32(gate[i])));
      o[i] = from_f32<T>(a);
    }
  }
}

template <typename T, int VPL, int GP>
static int launch_group(const void* q, int q_row_stride, const void* pages, const int* block_table, int max_pages,
                        int page_size, int num_pages, const int* positions, const int* token_req, void* out, int T_,
                        int nq, int nkv, int Dk, float scale, int window, int keep_first, int one_more, int vec,
                        ScoreShape shape, int* status, cudaStream_t stream) {
  const size_t smem = ((size_t)GP * Dk + (size_t)kGroupWarps * GP * (VPL * 32 + 2)) * sizeof(float);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(window_attention_group_kernel<T, VPL, GP>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  kvb_launch(window_attention_group_kernel<T, VPL, GP>, dim3(T_, nkv), dim3(kGroupWarps * 32), smem, stream, (const T*)q,
             q_row_stride, (const T*)pages, block_table, max_pages, page_size, num_pages, positions, token_req, (T*)out, nq,
             nkv, Dk, scale, window, keep_first, one_more, vec, shape, status);
  return kvb_launch_result();
}

template <typename T, int VPL>
static int launch_group_gp(int G, const void* q, int q_row_stride, const void* pages, const int* block_table,
                           int max_pages, int page_size, int num_pages, const int* positions, const int* token_req,
                           void* out, int T_, int nq, int nkv, int Dk, float scale, int window, int keep_first,
                           int one_more, int vec, ScoreShape shape, int* status, cudaStream_t stream) {
#define KVB_WG(GP) return launch_group<T, VPL, GP>(q, q_row_stride, pages, block_table, max_pages, page_size, num_pages, \
                                                   positions, token_req, out, T_, nq, nkv, Dk, scale, window, keep_first, \
                                                   one_more, vec, shape, status, stream)
  if (G == 1) KVB_WG(1);
  if (G == 2) KVB_WG(2);
  if (G <= 4) KVB_WG(4);
  KVB_WG(8);
#undef KVB_WG
}

// q points at the first query head of token 0; consecutive tokens are q_row_stride elements apart.
// pages: [num_pages, nkv, page_size, Dk + Dv].  out is [T, nq * Dv], dense.
// Refuses: Dk or Dv above 256, nq not a multiple of nkv, a negative window or keep_first.
static int window_attention_any(const void* q, int q_row_stride, const void* pages, const int* block_table,
                                int max_pages, int page_size, int num_pages, const int* positions,
                                const int* token_req, void* out, int T_, int nq, int nkv, int Dk, int Dv,
                                float scale, int window, int keep_first, int one_more, ScoreShape shape, int dtype,
                                int* status, cudaStream_t stream) {
  if (T_ <= 0) return 0;
  if (Dk > kMaxDim || Dv > kMaxDim || Dk < 1 || Dv < 1 || nkv < 1 || nq % nkv || window < 0 || keep_first < 0)
    return KVB_ERR_BAD_SIZE;
  if (shape.chunk < 0 || (shape.chunk > 0 && keep_first > 0) || (one_more && shape.sinks != nullptr)) return KVB_ERR_BAD_SIZE;
  const int esz = dtype == KVB_F32 ? 4 : 2;
  const int per16 = 16 / esz;
  const int vec = (Dk % per16 == 0 && (Dk + Dv) % per16 == 0 && ((uintptr_t)pages % 16) == 0) ? 1 : 0;
  // groups of up to 8 heads with values of 32, 64 or 128 channels: a block per key/value head, the rows read once
  const int G = nq / nkv;
  if (G <= kMaxGroup && (Dv == 32 || Dv == 64 || Dv == 128) && vec) {
#define KVB_WV(VPL)                                                                                                     \
  KVB_DISPATCH_DTYPE(dtype, T, return (launch_group_gp<T, VPL>(G, q, q_row_stride, pages, block_table, max_pages,      \
                                                               page_size, num_pages, positions, token_req, out, T_, nq, \
                                                               nkv, Dk, scale, window, keep_first, one_more, vec,      \
                                                               shape, status, stream)))
    if (Dv == 32) { KVB_WV(1); }
    if (Dv == 64) { KVB_WV(2); }
    if (Dv == 128) { KVB_WV(4); }
#undef KVB_WV
  }
  dim3 grid(T_, nq);
  KVB_DISPATCH_DTYPE(dtype, T, (kvb_launch(window_attention_kernel<T>, grid, dim3(kWarps * 32), 0, stream, (const T*)q,
                                            q_row_stride, (const T*)pages, block_table, max_pages, page_size, num_pages,
                                            positions, token_req, (T*)out, nq, nkv, Dk, Dv, scale, window, keep_first,
                                            one_more, vec, shape, status)));
  return kvb_launch_result();
}

KVB_EXPORT int kvb_window_attention(const void* q, int q_row_stride, const void* pages, const int* block_table,
                                    int max_pages, int page_size, int num_pages, const int* positions,
                                    const int* token_req, void* out, int T_, int nq, int nkv, int Dk, int Dv,
                                    float scale, int window, int keep_first, int one_more, int dtype, int* status,
                                    cudaStream_t stream) {
  const ScoreShape plain = {nullptr, nullptr, 0.f, 1.f};
  return window_attention_any(q, q_row_stride, pages, block_table, max_pages, page_size, num_pages, positions, token_req,
                              out, T_, nq, nkv, Dk, Dv, scale, window, keep_first, one_more, plain, dtype, status, stream);
}

// The same with the scores shaped on their way to the softmax (see ScoreShape): head_scale and slopes are
// float32 [nq] or null, softcap 0 for none, out_scale multiplies the result.
KVB_EXPORT int kvb_window_attention_shaped(const void* q, int q_row_stride, const void* pages, const int* block_table,
                                           int max_pages, int page_size, int num_pages, const int* positions,
                                           const int* token_req, void* out, int T_, int nq, int nkv, int Dk, int Dv,
                                           float scale, int window, int keep_first, int one_more,
                                           const float* head_scale, const float* slopes, float softcap, float out_scale,
                                           int dtype, int* status, cudaStream_t stream) {
  if (softcap < 0.f) return KVB_ERR_BAD_SIZE;
  const ScoreShape shape = {head_scale, slopes, softcap, out_scale};
  return window_attention_any(q, q_row_stride, pages, block_table, max_pages, page_size, num_pages, positions, token_req,
                              out, T_, nq, nkv, Dk, Dv, scale, window, keep_first, one_more, shape, dtype, status, stream);
}

// The same with everything a ScoreShape can say: also a learned score per head in the denominator (sinks, float32
// [nq] or null), a mask by blocks of `chunk` positions (0: none; not together with keep_first) and an output gate
// (gate: activations' type, [T, >= nq * Dv] with row stride gate_ld, or null).
KVB_EXPORT int kvb_window_attention_masked(const void* q, int q_row_stride, const void* pages, const int* block_table,
                                           int max_pages, int page_size, int num_pages, const int* positions,
                                           const int* token_req, void* out, int T_, int nq, int nkv, int Dk, int Dv,
                                           float scale, int window, int keep_first, int one_more,
                                           const float* head_scale, const float* slopes, float softcap, float out_scale,
                                           const float* sinks, int chunk, const void* gate, int gate_ld, int dtype,
                                           int* status, cudaStream_t stream) {
  if (softcap < 0.f) return KVB_ERR_BAD_SIZE;
  const ScoreShape shape = {head_scale, slopes, softcap, out_scale, sinks, chunk, gate, gate_ld};
  return window_attention_any(q, q_row_stride, pages, block_table, max_pages, page_size, num_pages, positions, token_req,
                              out, T_, nq, nkv, Dk, Dv, scale, window, keep_first, one_more, shape, dtype, status, stream);
}

// ---------------------------------------------------------------- biases, norms over the whole projection, rotation, cache write
// src [T, ld] holds, per token, nq queries of Dk from column 0, nkv keys of Dk from k_off and nkv values of Dv from
// v_off, as a product left them.  Each gets its bias (float32, may be null).  With qw (float32 [nq * Dk]) all of a
// token's queries together are divided by their root mean square (eps inside the root) and multiplied by qw, before
// they are cut into heads; the keys likewise with kw [nkv * Dk].  Then the first `rot` channels of every query and key
// head turn by the token's position: channel pair i is (i, i + rot / 2) with layout 0 and (2 i, 2 i + 1) with layout
// 1, and (u, v) becomes (u c - v s, v c + u s) with c = cos_t[pos][i], s = sin_t[pos][i] (float32 tables of
// table_len rows, rot / 2 wide; any factor on the rotation is in the tables).  Queries go to q_out [T, nq * Dk];
// keys and values into the request's pages, a row [key | value] per token and key/value head.  One block per token;
// the token's queries and keys wait in shared memory as float32 between the steps.
struct QkRotArgs {
  const void* src; int ld, k_off, v_off;
  const float* bq; const float* bk; const float* bv;
  const float* qw; const float* kw; float eps;
  const float* cos_t; const float* sin_t; int table_len, rot, layout;
  void* q_out; void* pages;
  const int* block_table; int max_pages, page_size, num_pages;
  const int* positions; const int* token_req;
  int nq, nkv, Dk, Dv, write;
  int* status;
};

__device__ __forceinline__ float turned(const float* x, int d, int rot, int layout, const float* c, const float* s) {
  if (d >= rot) return x[d];
  const int half = rot >> 1;
  if (layout == 0) {
    return d < half ? x[d] * c[d] - x[d + half] * s[d] : x[d] * c[d - half] + x[d - half] * s[d - half];
  }
  const int i = d >> 1;
  return (d & 1) == 0 ? x[d] * c[i] - x[d + 1] * s[i] : x[d] * c[i] + x[d - 1] * s[i];
}

template <typename T>
__global__ void __launch_bounds__(256) qk_rot_append_kernel(QkRotArgs a) {
  extern __shared__ float qk_s[];             // [nq * Dk] queries, then [nkv * Dk] keys
  __shared__ float part[2][8];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nQ = a.nq * a.Dk, nK = a.nkv * a.Dk, nV = a.nkv * a.Dv;
  float* ks = qk_s + nQ;
  const T* row = static_cast<const T*>(a.src) + (size_t)t * a.ld;
  const int pos = a.positions[t];
  float sq = 0.f, sk = 0.f;
  for (int i = threadIdx.x; i < nQ; i += blockDim.x) {
    const float v = to_f32(row[i]) + (a.bq ? a.bq[i] : 0.f);
    qk_s[i] = v;
    sq = fmaf(v, v, sq);
  }
  for (int i = threadIdx.x; i < nK; i += blockDim.x) {
    const float v = to_f32(row[a.k_off + i]) + (a.bk ? a.bk[i] : 0.f);
    ks[i] = v;
    sk = fmaf(v, v, sk);
  }
  sq = warp_sum(sq);
  sk = warp_sum(sk);
  if (lane == 0) { part[0][warp] = sq; part[1][warp] = sk; }
  __syncthreads();
  float tq = 0.f, tk = 0.f;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) { tq += part[0][w]; tk += part[1][w]; }
  if (a.qw != nullptr) {
    const float r = 1.0f / sqrtf(tq / (float)nQ + a.eps);
    for (int i = threadIdx.x; i < nQ; i += blockDim.x) qk_s[i] = qk_s[i] * r * a.qw[i];
  }
  if (a.kw != nullptr) {
    const float r = 1.0f / sqrtf(tk / (float)nK + a.eps);
    for (int i = threadIdx.x; i < nK; i += blockDim.x) ks[i] = ks[i] * r * a.kw[i];
  }
  __syncthreads();
  int rot = a.rot;
  const float* c = nullptr;
  const float* s = nullptr;
  if (rot > 0) {
    if (pos < 0 || pos >= a.table_len) {
      if (threadIdx.x == 0) atomicCAS(a.status, 0, KVB_STATUS_BAD_POSITION);
      rot = 0;
    } else {
      c = a.cos_t + (size_t)pos * (a.rot >> 1);
      s = a.sin_t + (size_t)pos * (a.rot >> 1);
    }
  }
  T* q_out = static_cast<T*>(a.q_out) + (size_t)t * nQ;
  for (int i = threadIdx.x; i < nQ; i += blockDim.x) {
    const int head = i / a.Dk, d = i - head * a.Dk;
    q_out[i] = from_f32<T>(turned(qk_s + head * a.Dk, d, rot, a.layout, c, s));
  }
  if (!a.write) return;
  const int lp = pos / a.page_size;
  const int page = (pos >= 0 && lp < a.max_pages) ? a.block_table[(size_t)a.token_req[t] * a.max_pages + lp] : -1;
  if (page < 0 || page >= a.num_pages) {
    if (threadIdx.x == 0) atomicCAS(a.status, 0, KVB_STATUS_UNMAPPED_PAGE);
    return;
  }
  T* pages = static_cast<T*>(a.pages);
  const int row_len = a.Dk + a.Dv;
  for (int i = threadIdx.x; i < nK; i += blockDim.x) {
    const int head = i / a.Dk, d = i - head * a.Dk;
    pages[(((size_t)page * a.nkv + head) * a.page_size + (pos % a.page_size)) * row_len + d] =
        from_f32<T>(turned(ks + head * a.Dk, d, rot, a.layout, c, s));
  }
  for (int i = threadIdx.x; i < nV; i += blockDim.x) {
    const int head = i / a.Dv, d = i - head * a.Dv;
    pages[(((size_t)page * a.nkv + head) * a.page_size + (pos % a.page_size)) * row_len + a.Dk + d] =
        from_f32<T>(to_f32(row[a.v_off + i]) + (a.bv ? a.bv[i] : 0.f));
  }
}

// Refuses: head sizes above 256, rot odd or above Dk, a layout other than 0 or 1, more than 48 K queries and keys a token.
KVB_EXPORT int kvb_qk_rot_append(const QkRotArgs* args, int T_, int dtype, cudaStream_t stream) {
  if (T_ <= 0) return 0;
  const QkRotArgs a = *args;
  if (a.Dk > kMaxDim || a.Dv > kMaxDim || a.Dk < 1 || a.Dv < 1 || a.nkv < 1 || a.nq < 1) return KVB_ERR_BAD_SIZE;
  if (a.rot < 0 || a.rot > a.Dk || (a.rot & 1) || a.layout < 0 || a.layout > 1) return KVB_ERR_BAD_SIZE;
  if (a.rot > 0 && (a.cos_t == nullptr || a.sin_t == nullptr)) return KVB_ERR_BAD_SIZE;
  const size_t smem = (size_t)(a.nq + a.nkv) * a.Dk * sizeof(float);
  if (smem > 192 * 1024) return KVB_ERR_BAD_SIZE;
  KVB_DISPATCH_DTYPE(dtype, T, {
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(qk_rot_append_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
    }
    kvb_launch(qk_rot_append_kernel<T>, dim3(T_), dim3(256), smem, stream, a);
  });
  return kvb_launch_result();
}

// ---------------------------------------------------------------- biases, per-head norms and the cache write
// src [T, ld] holds, per token, nq queries of Dk from column 0, nkv keys of Dk from k_off and nkv values of Dv from
// v_off, as a product left them.  Each gets its bias (float32, may be null); every query and key head is then
// divided by its root mean square (eps inside the root) and multiplied by a weight of Dk shared by the heads
// (qw, kw; null: no norm).  Queries go to q_out [T, nq * Dk]; keys and values into the request's pages, a row
// [key | value] per token and key/value head.  One block per token, a warp per head.
template <typename T>
__global__ void __launch_bounds__(256)
qk_norm_append_kernel(const T* __restrict__ src, int ld, int k_off, int v_off, const float* __restrict__ bq,
                      const float* __restrict__ bk, const float* __restrict__ bv, const float* __restrict__ qw,
                      const float* __restrict__ kw, float eps, T* __restrict__ q_out, T* __restrict__ pages,
                      const int* __restrict__ block_table, int max_pages, int page_size, int num_pages,
                      const int* __restrict__ positions, const int* __restrict__ token_req, int nq, int nkv, int Dk,
                      int Dv, int write, int* status) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const T* row = src + (size_t)t * ld;
  const int pos = positions[t];
  const int lp = pos / page_size;
  int page = -1;
  if (write) {
    page = lp < max_pages ? block_table[(size_t)token_req[t] * max_pages + lp] : -1;
    if (page < 0 || page >= num_pages) {
      if (threadIdx.x == 0) atomicCAS(status, 0, KVB_STATUS_UNMAPPED_PAGE);
      page = -1;
    }
  }
  for (int unit = warp; unit < nq + 2 * nkv; unit += nw) {
    const bool is_q = unit < nq, is_k = !is_q && unit < nq + nkv;
    const int head = is_q ? unit : (is_k ? unit - nq : unit - nq - nkv);
    const int D = (is_q || is_k) ? Dk : Dv;
    const T* x = row + (is_q ? head * Dk : (is_k ? k_off + head * Dk : v_off + head * Dv));
    const float* bias = is_q ? bq : (is_k ? bk : bv);
    const float* w = is_q ? qw : (is_k ? kw : nullptr);
    T* dst;
    if (is_q) {
      dst = q_out + ((size_t)t * nq + head) * Dk;
    } else {
      if (page < 0) continue;
      dst = pages + (((size_t)page * nkv + head) * page_size + (pos % page_size)) * (Dk + Dv) + (is_k ? 0 : Dk);
    }
    float v[kMaxDim / 32];
    float sq = 0.f;
#pragma unroll
    for (int r = 0; r < kMaxDim / 32; ++r) {
      const int i = r * 32 + lane;
      v[r] = 0.f;
      if (i < D) {
        v[r] = to_f32(x[i]) + (bias ? bias[head * D + i] : 0.f);
        sq = fmaf(v[r], v[r], sq);
      }
    }
    float f = 1.f;
    if (w != nullptr) f = 1.0f / sqrtf(warp_sum(sq) / (float)D + eps);
#pragma unroll
    for (int r = 0; r < kMaxDim / 32; ++r) {
      const int i = r * 32 + lane;
      if (i < D) dst[i] = from_f32<T>(w != nullptr ? v[r] * f * w[i] : v[r]);
    }
  }
}

KVB_EXPORT int kvb_qk_norm_append(const void* src, int ld, int k_off, int v_off, const float* bq, const float* bk,
                                  const float* bv, const float* qw, const float* kw, float eps, void* q_out, void* pages,
                                  const int* block_table, int max_pages, int page_size, int num_pages,
                                  const int* positions, const int* token_req, int T_, int nq, int nkv, int Dk, int Dv,
                                  int write, int dtype, int* status, cudaStream_t stream) {
  if (T_ <= 0) return 0;
  if (Dk > kMaxDim || Dv > kMaxDim || Dk < 1 || Dv < 1 || nkv < 1 || nq < 1) return KVB_ERR_BAD_SIZE;
  const int units = nq + 2 * nkv;
  const int threads = units >= 8 ? 256 : 32 * units;
  KVB_DISPATCH_DTYPE(dtype, T, (kvb_launch(qk_norm_append_kernel<T>, dim3(T_), dim3(threads), 0, stream, (const T*)src, ld,
                                            k_off, v_off, bq, bk, bv, qw, kw, eps, (T*)q_out, (T*)pages, block_table,
                                            max_pages, page_size, num_pages, positions, token_req, nq, nkv, Dk, Dv, write,
                                            status)));
  return kvb_launch_result();
}
