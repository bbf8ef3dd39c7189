// A matrix memory per head with exponential gates, kept stable by a running maximum (the mLSTM cell):
//
//   m_t = max(f_t + m_{t-1}, i_t)
//   C_t = exp(f_t + m_{t-1} - m_t) C_{t-1} + exp(i_t - m_t) k_t v_t^T        C is N x Dv
//   n_t = exp(f_t + m_{t-1} - m_t) n_{t-1} + exp(i_t - m_t) k_t
//   y_t = C_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)
//
// with i_t = cap tanh((a_t + b_i) / cap) and f_t = logsigmoid(cap tanh((b_t + b_f) / cap)) from the raw gate products
// a_t, b_t (float32).  C, n and m start at zero for a request that starts at position 0 (m at 0, not at minus
// infinity) and live in the request's state slot as float32.  Gates, their logarithms, the exponentials, the state and
// the read-out's denominator are float32 whatever the activations' type.
//
//   mlstm_scan        the recurrence along every request's run of tokens, y in float32
//   head_norm_gate    every head of y divided by its own root mean square, times a weight, times sigmoid(gate)
//
// mlstm_scan: a block owns up to 64 value columns of one (request, head); four lanes share a column, lane l holding
// the memory's rows l, l + 4, ... in registers for the whole run (rows 16 j + 4 l .. + 3 where N is a multiple of 4,
// so that one shared-memory load brings four rows of k or q).  Every thread also keeps its rows of n.  Where a head's
// columns are spread over several blocks (Dv above 64), each block keeps n and m for itself: the slot holds them once
// per block, so that no block reads what another has written.  The run is walked in pieces of 32 tokens whose q, k, v
// the block first brings into shared memory as float32; the piece's maxima m_t come from two scans across a warp
// (m_t = F_t + max(m before the piece, max_{s <= t}(i_s - F_s)), F the running sum of f inside the piece).
//
// A long run is cut into chunks of `chunk` tokens that are walked side by side, in three launches:
//   LOCAL   every chunk but a run's last, from an empty memory whose maximum starts at minus infinity: what it ends
//           with (C, n, m) and the sum of its f
//   carry   per element, along the run's chunks in order: what each chunk begins with
//           (m' = max(F + m, m_c);  C' = exp(F + m - m') C + exp(m_c - m') C_c)
//   FINAL   every chunk from what it begins with, writing y; the run's last chunk leaves the state in the slot
// A run of one chunk reads and writes its slot directly.
#include "common.cuh"

#include <math_constants.h>

struct MlstmArgs {
  const void* qkv; int ld; int q_off, k_off, v_off;   // [T, >= ...] activations' type: H x N queries, H x N keys, H x Dv values
  const float* gates; int ld_g;                        // [T, >= 2 H] float32: raw input gates, then raw forget gates
  const float* bi; const float* bf;                    // [H]
  float cap, q_scale;
  float* state; long long slot_stride;                 // slot 0's [H][Dv][N] | [H][splits][N] | [H][splits]
  float* y;                                            // [T, H * Dv] float32
  const int* q_start; const int* req_start; const int* slots;
  int H, N, Dv;
  int chunk, row_off;                                  // chunk > 0: runs are cut; requests below row_off are single chunks
  float* local; float* carry;                          // chunked: [rows][per] twice, per = the floats of one slot
  float* fsum;                                         // chunked: [rows][H] the chunks' sums of f
};

constexpr int kMlPiece = 32;
constexpr int kMlCols = 64;
enum { ML_WHOLE = 0, ML_LOCAL = 1, ML_FINAL = 2 };

__host__ __device__ __forceinline__ int ml_splits(int Dv) { return (Dv + kMlCols - 1) / kMlCols; }
// floats of one request's state: the matrices, then n and m once per block of columns
__host__ __device__ __forceinline__ size_t ml_state_floats(int H, int N, int Dv) {
  return (size_t)H * Dv * N + (size_t)H * ml_splits(Dv) * (N + 1);
}

__device__ __forceinline__ float log_sigmoid_f(float x) {
  return fminf(x, 0.f) - log1pf(expf(-fabsf(x)));
}

template <typename T, int NPT, int MODE, bool VEC>
__global__ void __launch_bounds__(256) mlstm_scan_kernel(MlstmArgs p) {
  extern __shared__ __align__(16) float msm[];
  const int N = p.N;
  float* ks = msm;                           // [piece][N]
  float* qs = ks + kMlPiece * N;             // [piece][N]
  float* vs = qs + kMlPiece * N;             // [piece][kMlCols]
  float* keep_s = vs + kMlPiece * kMlCols;   // [piece] exp(f + m_{t-1} - m_t)
  float* take_s = keep_s + kMlPiece;         // [piece] exp(i - m_t)
  float* em_s = take_s + kMlPiece;           // [piece] exp(-m_t)
  float* m_s = em_s + kMlPiece;              // [2]: m before the piece, the chunk's sum of f
  pdl_trigger();
  pdl_wait();
  const int splits = ml_splits(p.Dv);
  const int h = blockIdx.x / splits, sp = blockIdx.x % splits, col0 = sp * kMlCols;
  const int r = blockIdx.y;
  const int my_cols = min(kMlCols, p.Dv - col0);
  const int tid = threadIdx.x, l = tid & 3, pcol = tid >> 2;
  const bool owner = pcol < my_cols;
  const int pc = owner ? pcol : 0;
  int t0 = p.q_start[r], t1 = p.q_start[r + 1];
  const size_t mats = (size_t)p.H * p.Dv * N;
  const size_t at_c = ((size_t)h * p.Dv + col0 + pc) * N;                  // this thread's column
  const size_t at_n = mats + ((size_t)h * splits + sp) * N;               // this block's n
  const size_t at_m = mats + (size_t)p.H * splits * N + (size_t)h * splits + sp;
  float* slot = p.state + (size_t)p.slots[r] * p.slot_stride;
  const float* from = slot;                  // where the state comes from, null for an empty one
  float* to = slot;                          // where it goes, null for nowhere
  if (p.req_start[r] == 0) from = nullptr;
  float m0 = 0.f;                            // the maximum an empty memory starts with
  size_t row = 0;
  if (MODE != ML_WHOLE) {
    const int mine = t0 + (int)blockIdx.z * p.chunk;
    const bool single = t0 + p.chunk >= t1;                                // a run of one chunk
    if (MODE == ML_LOCAL ? mine + p.chunk >= t1 : (mine >= t1 && blockIdx.z > 0)) return;
    row = (size_t)(r - p.row_off) + mine / p.chunk;
    const size_t per = ml_state_floats(p.H, N, p.Dv);
    if (MODE == ML_LOCAL) { from = nullptr; to = p.local + row * per; m0 = -CUDART_INF_F; }
    else if (!single) { from = p.carry + row * per; to = mine + p.chunk >= t1 ? slot : nullptr; }
    t0 = mine;
    t1 = min(t1, mine + p.chunk);
  }
  float C[NPT], nv[NPT];
#pragma unroll
  for (int i = 0; i < NPT; ++i) {
    const int n = VEC ? 16 * (i >> 2) + 4 * l + (i & 3) : l + 4 * i;
    C[i] = (from && owner && n < N) ? from[at_c + n] : 0.f;
    nv[i] = (from && n < N) ? from[at_n + n] : 0.f;
  }
  if (tid == 0) { m_s[0] = from ? from[at_m] : m0; m_s[1] = 0.f; }
  const T* qkv = static_cast<const T*>(p.qkv);
  const float bi = p.bi ? p.bi[h] : 0.f, bf = p.bf ? p.bf[h] : 0.f;
  for (int c0 = t0; c0 < t1; c0 += kMlPiece) {
    const int nt = min(kMlPiece, t1 - c0);
    __syncthreads();
    for (int idx = tid; idx < nt * N; idx += blockDim.x) {
      const int tk = idx / N, n = idx - tk * N;
      const T* rowp = qkv + (size_t)(c0 + tk) * p.ld;
      ks[idx] = to_f32(rowp[p.k_off + h * N + n]);
      if (MODE != ML_LOCAL) qs[idx] = to_f32(rowp[p.q_off + h * N + n]) * p.q_scale;
    }
    for (int idx = tid; idx < nt * my_cols; idx += blockDim.x) {
      const int tk = idx / my_cols, q = idx - tk * my_cols;
      vs[tk * kMlCols + q] = to_f32(qkv[(size_t)(c0 + tk) * p.ld + p.v_off + h * p.Dv + col0 + q]);
    }
    if (tid < 32) {
      // the piece's gates and maxima: lane t is token t
      float gi = -CUDART_INF_F, gf = 0.f;
      if (tid < nt) {
        const float* g = p.gates + (size_t)(c0 + tid) * p.ld_g;
        gi = p.cap * tanhf((g[h] + bi) / p.cap);
        gf = log_sigmoid_f(p.cap * tanhf((g[p.H + h] + bf) / p.cap));
      }
      float F = gf;                               // running sum of f
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float x = __shfl_up_sync(0xffffffffu, F, o);
        if (tid >= o) F += x;
      }
      float G = gi - F;                           // running maximum of i_s - F_s
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float x = __shfl_up_sync(0xffffffffu, G, o);
        if (tid >= o) G = fmaxf(G, x);
      }
      const float mb = m_s[0];
      const float m = F + fmaxf(mb, G);
      float mp = __shfl_up_sync(0xffffffffu, m, 1);
      if (tid == 0) mp = mb;
      // from an empty memory whose maximum is minus infinity nothing is kept
      keep_s[tid] = mp == -CUDART_INF_F ? 0.f : expf(gf + mp - m);
      take_s[tid] = expf(gi - m);
      em_s[tid] = expf(-m);
      __syncwarp();
      if (tid == nt - 1) { m_s[0] = m; m_s[1] += F; }
    }
    __syncthreads();
    for (int tk = 0; tk < nt; ++tk) {
      const float kp = keep_s[tk], tkk = take_s[tk];
      const float w = tkk * vs[tk * kMlCols + pc];
      const float* kt = ks + tk * N;
      if (MODE == ML_LOCAL) {
        if (VEC) {
#pragma unroll
          for (int j = 0; j < NPT / 4; ++j) {
            const int n = 16 * j + 4 * l;
            if (n < N) {
              const float4 kv = *reinterpret_cast<const float4*>(kt + n);
              C[4 * j + 0] = fmaf(kp, C[4 * j + 0], w * kv.x); nv[4 * j + 0] = fmaf(kp, nv[4 * j + 0], tkk * kv.x);
              C[4 * j + 1] = fmaf(kp, C[4 * j + 1], w * kv.y); nv[4 * j + 1] = fmaf(kp, nv[4 * j + 1], tkk * kv.y);
              C[4 * j + 2] = fmaf(kp, C[4 * j + 2], w * kv.z); nv[4 * j + 2] = fmaf(kp, nv[4 * j + 2], tkk * kv.z);
              C[4 * j + 3] = fmaf(kp, C[4 * j + 3], w * kv.w); nv[4 * j + 3] = fmaf(kp, nv[4 * j + 3], tkk * kv.w);
            }
          }
        } else {
#pragma unroll
          for (int i = 0; i < NPT; ++i) {
            const int n = l + 4 * i;
            if (n < N) { C[i] = fmaf(kp, C[i], w * kt[n]); nv[i] = fmaf(kp, nv[i], tkk * kt[n]); }
          }
        }
        continue;
      }
      const float* qt = qs + tk * N;
      float acc = 0.f, den = 0.f;
      if (VEC) {
        float a1 = 0.f, d1 = 0.f;
#pragma unroll
        for (int j = 0; j < NPT / 4; ++j) {
          const int n = 16 * j + 4 * l;
          if (n < N) {
            const float4 kv = *reinterpret_cast<const float4*>(kt + n);
            const float4 qv = *reinterpret_cast<const float4*>(qt + n);
            C[4 * j + 0] = fmaf(kp, C[4 * j + 0], w * kv.x); nv[4 * j + 0] = fmaf(kp, nv[4 * j + 0], tkk * kv.x);
            C[4 * j + 1] = fmaf(kp, C[4 * j + 1], w * kv.y); nv[4 * j + 1] = fmaf(kp, nv[4 * j + 1], tkk * kv.y);
            C[4 * j + 2] = fmaf(kp, C[4 * j + 2], w * kv.z); nv[4 * j + 2] = fmaf(kp, nv[4 * j + 2], tkk * kv.z);
            C[4 * j + 3] = fmaf(kp, C[4 * j + 3], w * kv.w); nv[4 * j + 3] = fmaf(kp, nv[4 * j + 3], tkk * kv.w);
            acc = fmaf(C[4 * j + 0], qv.x, acc); den = fmaf(nv[4 * j + 0], qv.x, den);
            a1 = fmaf(C[4 * j + 1], qv.y, a1); d1 = fmaf(nv[4 * j + 1], qv.y, d1);
            acc = fmaf(C[4 * j + 2], qv.z, acc); den = fmaf(nv[4 * j + 2], qv.z, den);
            a1 = fmaf(C[4 * j + 3], qv.w, a1); d1 = fmaf(nv[4 * j + 3], qv.w, d1);
          }
        }
        acc += a1;
        den += d1;
      } else {
#pragma unroll
        for (int i = 0; i < NPT; ++i) {
          const int n = l + 4 * i;
          if (n < N) {
            C[i] = fmaf(kp, C[i], w * kt[n]);
            nv[i] = fmaf(kp, nv[i], tkk * kt[n]);
            acc = fmaf(C[i], qt[n], acc);
            den = fmaf(nv[i], qt[n], den);
          }
        }
      }
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      den += __shfl_xor_sync(0xffffffffu, den, 1);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      den += __shfl_xor_sync(0xffffffffu, den, 2);
      if (owner && l == 0)
        p.y[(size_t)(c0 + tk) * p.H * p.Dv + h * p.Dv + col0 + pc] = acc / (fmaxf(fabsf(den), em_s[tk]) + 1e-6f);
    }
  }
  __syncthreads();
  if (to) {
#pragma unroll
    for (int i = 0; i < NPT; ++i) {
      const int n = VEC ? 16 * (i >> 2) + 4 * l + (i & 3) : l + 4 * i;
      if (n < N) {
        if (owner) to[at_c + n] = C[i];
        if (pcol == 0) to[at_n + n] = nv[i];
      }
    }
    if (tid == 0) to[at_m] = m_s[0];
  }
  if (MODE == ML_LOCAL && tid == 0 && sp == 0) p.fsum[row * p.H + h] = m_s[1];
}

// One thread per float of a request's state walks the run's chunks in order and writes what each begins with.
// Runs of one chunk are left alone.
__global__ void __launch_bounds__(256) mlstm_carry_kernel(MlstmArgs p) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.y;
  const int splits = ml_splits(p.Dv);
  const size_t mats = (size_t)p.H * p.Dv * p.N, vecs = (size_t)p.H * splits * p.N;
  const size_t per = mats + vecs + (size_t)p.H * splits;
  const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= per) return;
  const int t0 = p.q_start[r], t1 = p.q_start[r + 1];
  if (t0 + p.chunk >= t1) return;
  // the head this float belongs to, and where its block of columns keeps m
  int h, sp;
  if (e < mats) {
    h = (int)(e / ((size_t)p.Dv * p.N));
    sp = (int)((e / p.N) % p.Dv) / kMlCols;
  } else if (e < mats + vecs) {
    const size_t v = (e - mats) / p.N;
    h = (int)(v / splits); sp = (int)(v % splits);
  } else {
    const size_t v = e - mats - vecs;
    h = (int)(v / splits); sp = (int)(v % splits);
  }
  const size_t at_m = mats + vecs + (size_t)h * splits + sp;
  const bool is_m = e >= mats + vecs;
  const bool fresh = p.req_start[r] == 0;
  const float* slot = p.state + (size_t)p.slots[r] * p.slot_stride;
  float S = fresh ? 0.f : slot[e];
  float m = fresh ? 0.f : slot[at_m];
  const int nck = (t1 - t0 + p.chunk - 1) / p.chunk;
  const size_t row0 = (size_t)(r - p.row_off) + t0 / p.chunk;              // rows of one run follow one another
  for (int k = 0; k < nck; ++k) {
    p.carry[(row0 + k) * per + e] = is_m ? m : S;
    if (k + 1 == nck) break;
    const float F = p.fsum[(row0 + k) * p.H + h];
    const float mc = p.local[(row0 + k) * per + at_m];
    const float mn = fmaxf(F + m, mc);
    if (!is_m) S = expf(F + m - mn) * S + expf(mc - mn) * p.local[(row0 + k) * per + e];
    m = mn;
  }
}

KVB_EXPORT long long kvb_mlstm_state_floats(int H, int N, int Dv) { return (long long)ml_state_floats(H, N, Dv); }

// max_run: the step's longest run (chunked launches only: the grid's third extent).
// Refuses: N above 256, H or Dv below 1, a chunk that is no multiple of 32, more than 65535 requests or chunks.
KVB_EXPORT int kvb_mlstm_scan(const MlstmArgs* args, int R, int max_run, int dtype, cudaStream_t stream) {
  MlstmArgs p = *args;
  if (R <= 0) return 0;
  if (p.H < 1 || p.N < 1 || p.N > 256 || p.Dv < 1 || R > 65535 || !(p.cap > 0.f)) return KVB_ERR_BAD_SIZE;
  unsigned nck = 1;
  if (p.chunk > 0) {
    if (!p.local || !p.carry || !p.fsum || max_run < 1 || p.chunk % kMlPiece) return KVB_ERR_BAD_SIZE;
    nck = (unsigned)((max_run + p.chunk - 1) / p.chunk);
    if (nck > 65535) return KVB_ERR_BAD_SIZE;
  }
  const int splits = ml_splits(p.Dv);
  const int cols = p.Dv < kMlCols ? p.Dv : kMlCols;
  const int threads = (cols * 4 + 31) / 32 * 32;
  const size_t smem = ((size_t)kMlPiece * (2 * p.N + kMlCols) + 3 * kMlPiece + 2) * sizeof(float);
  const int npt = (p.N + 3) / 4;
  const dim3 grid(p.H * splits, R, nck);
#define KVB_ML_MODE(NPT, MODE, VEC)                                                                                  \
  {                                                                                                                \
    if (smem > 48 * 1024) {                                                                                        \
      cudaError_t e = cudaFuncSetAttribute(mlstm_scan_kernel<T, NPT, MODE, VEC>,                                   \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                \
      if (e != cudaSuccess) return (int)e;                                                                         \
    }                                                                                                              \
    kvb_launch(mlstm_scan_kernel<T, NPT, MODE, VEC>, grid, dim3(threads), smem, stream, p);                        \
  }
#define KVB_ML_VEC(MODE, VEC)                                                                                      \
  KVB_DISPATCH_DTYPE(dtype, T, {                                                                                   \
    if (npt <= 8) KVB_ML_MODE(8, MODE, VEC)                                                                        \
    else if (npt <= 16) KVB_ML_MODE(16, MODE, VEC)                                                                 \
    else if (npt <= 32) KVB_ML_MODE(32, MODE, VEC)                                                                 \
    else KVB_ML_MODE(64, MODE, VEC)                                                                                \
  })
#define KVB_ML(MODE)                                                                                               \
  {                                                                                                                \
    if (p.N % 4 == 0) KVB_ML_VEC(MODE, true) else KVB_ML_VEC(MODE, false)                                          \
  }
  if (p.chunk > 0) {
    KVB_ML(ML_LOCAL);
    const size_t per = ml_state_floats(p.H, p.N, p.Dv);
    kvb_launch(mlstm_carry_kernel, dim3((unsigned)((per + 255) / 256), R), dim3(256), 0, stream, p);
    KVB_ML(ML_FINAL);
  } else {
    KVB_ML(ML_WHOLE);
  }
#undef KVB_ML
#undef KVB_ML_VEC
#undef KVB_ML_MODE
  return kvb_launch_result();
}

// ---------------------------------------------------------------- a norm per head, a weight, a sigmoid gate
// y [T, heads * Dv] float32; gate [T, >= heads * Dv] activations' type with row stride ld_g; weight [heads * Dv] float32.
// out[t, c] = y / sqrt(mean over c's head of y^2 + eps) * weight[c] * sigmoid(gate[t, c]).  A warp per (token, head).
template <typename T>
__global__ void __launch_bounds__(256)
head_norm_gate_kernel(const float* __restrict__ y, const T* __restrict__ gate, int ld_g, const float* __restrict__ weight,
                      T* __restrict__ out, int total, int heads, int Dv, float eps) {
  pdl_trigger();
  pdl_wait();
  const int unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (unit >= total) return;
  const int lane = threadIdx.x & 31;
  const int t = unit / heads, h = unit - t * heads;
  const float* row = y + ((size_t)t * heads + h) * Dv;
  float ss = 0.f;
  for (int i = lane; i < Dv; i += 32) ss = fmaf(row[i], row[i], ss);
  const float r = 1.0f / sqrtf(warp_sum(ss) / (float)Dv + eps);
  const T* g = gate + (size_t)t * ld_g + (size_t)h * Dv;
  T* o = out + ((size_t)t * heads + h) * Dv;
  for (int i = lane; i < Dv; i += 32) {
    const float s = 1.0f / (1.0f + expf(-to_f32(g[i])));
    o[i] = from_f32<T>(row[i] * r * weight[h * Dv + i] * s);
  }
}

KVB_EXPORT int kvb_head_norm_gate(const float* y, const void* gate, int ld_g, const float* weight, void* out, int T_,
                                  int heads, int Dv, float eps, int dtype, cudaStream_t stream) {
  if (T_ <= 0) return 0;
  if (heads < 1 || Dv < 1) return KVB_ERR_BAD_SIZE;
  const long long total = (long long)T_ * heads;
  if (total > 0x7fffffffLL) return KVB_ERR_BAD_SIZE;
  KVB_DISPATCH_DTYPE(dtype, T, (kvb_launch(head_norm_gate_kernel<T>, dim3((unsigned)((total + 7) / 8)), dim3(256), 0, stream, y,
                                            (const T*)gate, ld_g, weight, (T*)out, (int)total, heads, Dv, eps)));
  return kvb_launch_result();
}
