// Mixers whose state is a linear recurrence with a decay that depends on the token.
//
//   gate_coeffs        the two gates of a diagonal recurrence from products with one square matrix per block of
//                      channels, turned at once into the recurrence's coefficients
//                          r = sigmoid(Wr_b u_b + br), i = sigmoid(Wi_b u_b + bi),
//                          log a = -c r softplus(lam),  a = exp(log a),  b = sqrt(1 - a^2) i u
//   diag_scan          S_t = a_t S_{t-1} + b_t per channel along each request's tokens, read out as
//                      S_t * gelu_tanh(y_t + bias) * out_scale; state [channels] per request slot
//   ssd_scan           a matrix state N x Dv per head with one decay per head and token:
//                          dt = softplus(dt_raw + dt_bias), S_t = exp(-exp(A_log) dt) S_{t-1} + dt B_t x_t^T,
//                          y_t = S_t^T C_t + D x_t
//   gated_group_norm   y * silu(z), then an RMS norm over each of `groups` equal parts of the row, times a weight
//
// Gates, decays, their logarithms, softplus, exponentials, step sizes and the states are float32 in both
// precisions.  A request that starts at position 0 starts from a zero state whatever its slot holds.  Sums run
// in an order fixed by the sizes alone, so a token's result does not depend on how its request was cut into
// steps or on the rest of the batch.
#include "common.cuh"

#include <math_constants.h>

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float gelu_tanh_f(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// ---------------------------------------------------------------- gates -> coefficients
// u [T, ld_u] (channels C = nb * bw); W [nb, 2 bw, bw]: rows 0 .. bw-1 of block b make r, rows bw .. 2bw-1 make i.
// a_out, b_out [T, C] float32.  Tiles of 64 tokens x 64 channels of one block, float32 sums in ascending k.
constexpr int GC_BM = 64, GC_BN = 64, GC_BK = 16;

template <typename T>
__global__ void __launch_bounds__(256)
gate_coeffs_kernel(const T* __restrict__ u, int ld_u, const T* __restrict__ W, const float* __restrict__ br,
                   const float* __restrict__ bi, const float* __restrict__ lam, float decay_scale,
                   float* __restrict__ a_out, float* __restrict__ b_out, int M, int bw, int C) {
  __shared__ float As[GC_BK][GC_BM + 4];
  __shared__ float Wr[GC_BK][GC_BN + 4];
  __shared__ float Wi[GC_BK][GC_BN + 4];
  pdl_trigger();
  pdl_wait();
  const int blk = blockIdx.z;
  const T* A = u + (size_t)blk * bw;
  const T* Wb = W + (size_t)blk * 2 * bw * bw;
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * GC_BM, n0 = blockIdx.x * GC_BN;
  const int tx = tid & 15, ty = tid >> 4;
  float ar[4][4], ai[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) { ar[i][j] = 0.f; ai[i][j] = 0.f; }
  const int lrow = tid >> 2, lk = (tid & 3) * 4;
  for (int k0 = 0; k0 < bw; k0 += GC_BK) {
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      const int k = k0 + lk + x;
      const int am = m0 + lrow, wn = n0 + lrow;
      As[lk + x][lrow] = (am < M && k < bw) ? to_f32(A[(size_t)am * ld_u + k]) : 0.f;
      Wr[lk + x][lrow] = (wn < bw && k < bw) ? to_f32(Wb[(size_t)wn * bw + k]) : 0.f;
      Wi[lk + x][lrow] = (wn < bw && k < bw) ? to_f32(Wb[(size_t)(bw + wn) * bw + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < GC_BK; ++kk) {
      float a[4], r[4], g[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) { r[j] = Wr[kk][tx * 4 + j]; g[j] = Wi[kk][tx * 4 + j]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) { ar[i][j] = fmaf(a[i], r[j], ar[i][j]); ai[i][j] = fmaf(a[i], g[j], ai[i][j]); }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= bw) continue;
      const int c = blk * bw + n;
      const float r = sigmoid_f(ar[i][j] + br[c]), g = sigmoid_f(ai[i][j] + bi[c]);
      const float la = -decay_scale * r * softplus_f(lam[c]);
      const float uv = to_f32(u[(size_t)m * ld_u + c]);
      a_out[(size_t)m * C + c] = expf(la);
      b_out[(size_t)m * C + c] = sqrtf(-expm1f(2.0f * la)) * g * uv;     // 1 - a^2 without cancellation near a = 1
    }
  }
}

KVB_EXPORT int kvb_gate_coeffs(const void* u, int ld_u, const void* W, const float* br, const float* bi,
                               const float* lam, float decay_scale, float* a_out, float* b_out, int M, int nb, int bw,
                               int dtype, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (nb < 1 || bw < 1 || nb > 65535) return KVB_ERR_BAD_SIZE;
  dim3 grid((bw + GC_BN - 1) / GC_BN, (M + GC_BM - 1) / GC_BM, nb);
  if (grid.y > 65535) return KVB_ERR_BAD_SIZE;
  KVB_DISPATCH_DTYPE(dtype, T, (kvb_launch(gate_coeffs_kernel<T>, grid, dim3(256), 0, stream, (const T*)u, ld_u,
                                            (const T*)W, br, bi, lam, decay_scale, a_out, b_out, M, bw, nb * bw)));
  return kvb_launch_result();
}

// The same coefficients from gate sums that a matrix product has already made: pre [nb, T, 2 bw] float32
// (per block of channels and token the r sums, then the i sums).
template <typename T>
__global__ void coeffs_from_sums_kernel(const float* __restrict__ pre, const T* __restrict__ u, int ld_u,
                                        const float* __restrict__ br, const float* __restrict__ bi,
                                        const float* __restrict__ lam, float decay_scale, float* __restrict__ a_out,
                                        float* __restrict__ b_out, long long total, int bw, int C, int M) {
  pdl_trigger();
  pdl_wait();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const long long m = idx / C;
  const int c = (int)(idx - m * C);
  const int blk = c / bw, n = c - blk * bw;
  const float* p = pre + ((size_t)blk * M + m) * 2 * bw;
  const float r = sigmoid_f(p[n] + br[c]), g = sigmoid_f(p[bw + n] + bi[c]);
  const float la = -decay_scale * r * softplus_f(lam[c]);
  a_out[idx] = expf(la);
  b_out[idx] = sqrtf(-expm1f(2.0f * la)) * g * to_f32(u[(size_t)m * ld_u + c]);
}

KVB_EXPORT int kvb_coeffs_from_sums(const float* pre, const void* u, int ld_u, const float* br, const float* bi,
                                    const float* lam, float decay_scale, float* a_out, float* b_out, int M, int nb,
                                    int bw, int dtype, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (nb < 1 || bw < 1) return KVB_ERR_BAD_SIZE;
  const long long total = (long long)M * nb * bw;
  KVB_DISPATCH_DTYPE(dtype, T, (kvb_launch(coeffs_from_sums_kernel<T>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0,
                                            stream, pre, (const T*)u, ld_u, br, bi, lam, decay_scale, a_out, b_out, total,
                                            bw, nb * bw, M)));
  return kvb_launch_result();
}

// ---------------------------------------------------------------- diagonal recurrence
// One thread per (request, channel) walks the request's tokens of this step, four tokens' coefficients requested
// at a time; the chain itself is one multiply-add per token.
//
// A long run is cut into chunks of kDiagChunk tokens that are walked side by side.  A first kernel reduces every
// chunk but a run's last to the pair (A, B) with S_end = A S_begin + B and notes the run's starting state; the
// second walks chunk k from the state that the pairs of chunks 0 .. k-1 give when applied in order, and the run's
// last chunk leaves the state in the slot.  Request row r's chunk that begins at token row t of the step keeps its
// pair in row (r - row_off) + t / kDiagChunk of `sum_a`, `sum_b`: rows grow with r and with t, so no two chunks share one.
struct DiagArgs {
  const float* a; const float* b;        // [T, C]
  const void* y; int ld_y;               // [T, >= C] compute type, gate branch before its activation
  const float* y_bias;                   // [C] or null
  float out_scale;
  void* out;                             // [T, C] compute type
  float* state; long long slot_stride;   // slot 0's [C]
  const int* q_start; const int* req_start; const int* slots;
  int C;
  int chunked, row_off;                  // chunked: runs are cut; requests below row_off are single chunks
  float* sum_a; float* sum_b; float* begin;   // chunked: [rows, C] pairs, [R, C] starting states
};

constexpr int kDiagChunk = 64;

__global__ void __launch_bounds__(128) diag_chunk_pairs_kernel(DiagArgs p) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.y, k = blockIdx.z;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= p.C) return;
  const int run0 = p.q_start[r], run1 = p.q_start[r + 1];
  if (k == 0) p.begin[(size_t)r * p.C + c] = p.req_start[r] > 0 ? p.state[(size_t)p.slots[r] * p.slot_stride + c] : 0.f;
  const int t0 = run0 + k * kDiagChunk;
  if (t0 + kDiagChunk >= run1) return;                 // the run's last chunk (or beyond it): nobody reads its pair
  float A = 1.f, B = 0.f;
  for (int t = t0; t < t0 + kDiagChunk; t += 4) {
    float a[4], b[4];
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      a[x] = p.a[(size_t)(t + x) * p.C + c];
      b[x] = p.b[(size_t)(t + x) * p.C + c];
    }
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      B = fmaf(a[x], B, b[x]);
      A *= a[x];
    }
  }
  const size_t row = (size_t)(r - p.row_off) + t0 / kDiagChunk;
  p.sum_a[row * p.C + c] = A;
  p.sum_b[row * p.C + c] = B;
}

template <typename T>
__global__ void __launch_bounds__(128) diag_scan_kernel(DiagArgs p) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= p.C) return;
  int t0 = p.q_start[r], t1 = p.q_start[r + 1];
  float* st = p.state + (size_t)p.slots[r] * p.slot_stride;
  float S;
  bool last = true;
  if (p.chunked) {
    const int k = blockIdx.z, mine = t0 + k * kDiagChunk;
    if (mine >= t1 && k > 0) return;
    S = p.begin[(size_t)r * p.C + c];
    for (int j = 0; j < k; ++j) {
      const size_t row = (size_t)(r - p.row_off) + (t0 + j * kDiagChunk) / kDiagChunk;
      S = fmaf(p.sum_a[row * p.C + c], S, p.sum_b[row * p.C + c]);
    }
    t0 = mine;
    last = mine + kDiagChunk >= t1;
    t1 = min(t1, mine + kDiagChunk);
  } else {
    S = p.req_start[r] > 0 ? st[c] : 0.f;
  }
  const float yb = p.y_bias ? p.y_bias[c] : 0.f;
  const T* y = static_cast<const T*>(p.y);
  T* out = static_cast<T*>(p.out);
  int t = t0;
  for (; t + 4 <= t1; t += 4) {
    float a[4], b[4], g[4];
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      a[x] = p.a[(size_t)(t + x) * p.C + c];
      b[x] = p.b[(size_t)(t + x) * p.C + c];
      g[x] = to_f32(y[(size_t)(t + x) * p.ld_y + c]);
    }
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      S = fmaf(a[x], S, b[x]);
      out[(size_t)(t + x) * p.C + c] = from_f32<T>(S * gelu_tanh_f(g[x] + yb) * p.out_scale);
    }
  }
  for (; t < t1; ++t) {
    S = fmaf(p.a[(size_t)t * p.C + c], S, p.b[(size_t)t * p.C + c]);
    out[(size_t)t * p.C + c] = from_f32<T>(S * gelu_tanh_f(to_f32(y[(size_t)t * p.ld_y + c]) + yb) * p.out_scale);
  }
  if (last) st[c] = S;
}

KVB_EXPORT int kvb_diag_chunk() { return kDiagChunk; }

// max_run: the step's longest run (chunked launches only: the grid's third extent).
KVB_EXPORT int kvb_diag_scan(const DiagArgs* args, int R, int max_run, int dtype, cudaStream_t stream) {
  DiagArgs p = *args;
  if (R <= 0) return 0;
  if (p.C < 1 || R > 65535) return KVB_ERR_BAD_SIZE;
  dim3 grid((p.C + 127) / 128, R, 1);
  if (p.chunked) {
    if (!p.sum_a || !p.sum_b || !p.begin || max_run < 1) return KVB_ERR_BAD_SIZE;
    grid.z = (max_run + kDiagChunk - 1) / kDiagChunk;
    if (grid.z > 65535) return KVB_ERR_BAD_SIZE;
    kvb_launch(diag_chunk_pairs_kernel, grid, dim3(128), 0, stream, p);
  }
  KVB_DISPATCH_DTYPE(dtype, T, (kvb_launch(diag_scan_kernel<T>, grid, dim3(128), 0, stream, p)));
  return kvb_launch_result();
}

// ---------------------------------------------------------------- matrix state with a decay per head
// A block owns `cols` value columns of one (request, head); four lanes share a column, lane l holding state rows
// l, l + 4, ... (NPT of them) in registers for the whole run; where N is a multiple of 4 (VEC) the lane holds rows
// 16 j + 4 l .. + 3 instead, so that one shared-memory load brings four rows of B or C.  The run is walked in pieces
// of 32 tokens whose B, C, x and step sizes the block first brings into shared memory as float32.
//
// A long run is cut into chunks of `chunk` tokens that are walked side by side, in three launches:
//   SSD_LOCAL   every chunk but a run's last, from a zero state: the state it ends with and the product of its decays
//   ssd_carry   per state element, along the run's chunks in order: what each chunk begins with (S <- decay S + local)
//   SSD_FINAL   every chunk from what it begins with, writing y; the run's last chunk leaves the state in the slot
// Request row r's chunk that begins at token row t keeps its matrices in row (r - row_off) + t / chunk of `local`
// (what it ends with from zero) and of `carry` (what it begins with): two arrays, so that the middle launch's loads
// do not wait for its stores.
// A run of one chunk reads and writes its slot directly.
struct SsdArgs {
  const void* xbc; int ld_xbc;           // [T, >= inner + 2 G N] compute type: x | B | C behind the convolution
  const void* dt; int ld_dt;             // [T, >= H] compute type: raw step sizes
  const float* dt_bias; const float* A_log; const float* D;      // [H]
  float* state; long long slot_stride;   // slot 0's [H][Dv][N]
  float* y;                              // [T, H * Dv] float32
  const int* q_start; const int* req_start; const int* slots;
  int H, G, N, Dv, cols;
  int chunk, row_off;                    // chunk > 0: runs are cut; requests below row_off are single chunks
  float* local; float* carry; float* decay;   // chunked: [rows][H][Dv][N] twice and [rows][H]
};

constexpr int kSsdPiece = 32;
enum { SSD_WHOLE = 0, SSD_LOCAL = 1, SSD_FINAL = 2 };

template <typename T, int NPT, int MODE, bool VEC>
__global__ void __launch_bounds__(256) ssd_scan_kernel(SsdArgs p) {
  extern __shared__ __align__(16) float ssm[];
  const int N = p.N, cols = p.cols;
  float* Bs = ssm;                          // [piece][N]
  float* Cs = Bs + kSsdPiece * N;           // [piece][N]
  float* xs = Cs + kSsdPiece * N;           // [piece][cols]
  float* dts = xs + kSsdPiece * cols;       // [piece]
  float* das = dts + kSsdPiece;             // [piece]
  pdl_trigger();
  pdl_wait();
  const int splits = (p.Dv + cols - 1) / cols;
  const int h = blockIdx.x / splits, col0 = (blockIdx.x % splits) * cols;
  const int r = blockIdx.y;
  const int g = h / (p.H / p.G);
  const int inner = p.H * p.Dv;
  const int my_cols = min(cols, p.Dv - col0);
  const int tid = threadIdx.x, l = tid & 3;
  const int pcol = tid >> 2;
  const bool owner = pcol < my_cols;
  const int pc = owner ? pcol : 0;
  int t0 = p.q_start[r], t1 = p.q_start[r + 1];
  const size_t at = ((size_t)h * p.Dv + col0 + pc) * N;          // this thread's column within a set of matrices
  float* st = p.state + (size_t)p.slots[r] * p.slot_stride + at;
  const float* from = st;                   // where the state comes from, null for zeros
  float* to = st;                           // where it goes, null for nowhere
  if (p.req_start[r] == 0) from = nullptr;
  size_t row = 0;
  if (MODE != SSD_WHOLE) {
    const int mine = t0 + (int)blockIdx.z * p.chunk;
    const bool single = t0 + p.chunk >= t1;                      // a run of one chunk
    if (MODE == SSD_LOCAL ? mine + p.chunk >= t1 : (mine >= t1 && blockIdx.z > 0)) return;
    row = (size_t)(r - p.row_off) + mine / p.chunk;
    const size_t mat = row * (size_t)inner * N + at;
    if (MODE == SSD_LOCAL) { from = nullptr; to = p.local + mat; }
    else if (!single) { from = p.carry + mat; to = mine + p.chunk >= t1 ? st : nullptr; }
    t0 = mine;
    t1 = min(t1, mine + p.chunk);
  }
  float S[NPT];
#pragma unroll
  for (int i = 0; i < NPT; ++i) {
    const int n = VEC ? 16 * (i >> 2) + 4 * l + (i & 3) : l + 4 * i;
    S[i] = (from && owner && n < N) ? from[n] : 0.f;
  }
  const T* xbc = static_cast<const T*>(p.xbc);
  const T* dt = static_cast<const T*>(p.dt);
  const float rate = expf(p.A_log[h]), dskip = p.D[h], dtb = p.dt_bias[h];
  float shrink = 1.f;                       // SSD_LOCAL: the product of the chunk's decays
  for (int c0 = t0; c0 < t1; c0 += kSsdPiece) {
    const int nt = min(kSsdPiece, t1 - c0);
    __syncthreads();
    for (int idx = tid; idx < nt * N; idx += blockDim.x) {
      const int tk = idx / N, n = idx - tk * N;
      const T* rowp = xbc + (size_t)(c0 + tk) * p.ld_xbc + inner + g * N;
      Bs[idx] = to_f32(rowp[n]);
      if (MODE != SSD_LOCAL) Cs[idx] = to_f32(rowp[p.G * N + n]);
    }
    for (int idx = tid; idx < nt * my_cols; idx += blockDim.x) {
      const int tk = idx / my_cols, q = idx - tk * my_cols;
      xs[tk * cols + q] = to_f32(xbc[(size_t)(c0 + tk) * p.ld_xbc + h * p.Dv + col0 + q]);
    }
    if (tid < nt) {
      const float d = softplus_f(to_f32(dt[(size_t)(c0 + tid) * p.ld_dt + h]) + dtb);
      dts[tid] = d;
      das[tid] = expf(-rate * d);
    }
    __syncthreads();
    for (int tk = 0; tk < nt; ++tk) {
      const float xv = xs[tk * cols + pc];
      const float w = dts[tk] * xv, da = das[tk];
      const float* Bt = Bs + tk * N;
      if (MODE == SSD_LOCAL) {
        shrink *= da;
        if (VEC) {
#pragma unroll
          for (int j = 0; j < NPT / 4; ++j) {
            const int n = 16 * j + 4 * l;
            if (n < N) {
              const float4 bv = *reinterpret_cast<const float4*>(Bt + n);
              S[4 * j + 0] = fmaf(da, S[4 * j + 0], w * bv.x);
              S[4 * j + 1] = fmaf(da, S[4 * j + 1], w * bv.y);
              S[4 * j + 2] = fmaf(da, S[4 * j + 2], w * bv.z);
              S[4 * j + 3] = fmaf(da, S[4 * j + 3], w * bv.w);
            }
          }
        } else {
#pragma unroll
          for (int i = 0; i < NPT; ++i) {
            const int n = l + 4 * i;
            if (n < N) S[i] = fmaf(da, S[i], w * Bt[n]);
          }
        }
        continue;
      }
      const float* Ct = Cs + tk * N;
      float acc = 0.f;
      if (VEC) {
        float a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
        for (int j = 0; j < NPT / 4; ++j) {
          const int n = 16 * j + 4 * l;
          if (n < N) {
            const float4 bv = *reinterpret_cast<const float4*>(Bt + n);
            const float4 cv = *reinterpret_cast<const float4*>(Ct + n);
            S[4 * j + 0] = fmaf(da, S[4 * j + 0], w * bv.x);
            S[4 * j + 1] = fmaf(da, S[4 * j + 1], w * bv.y);
            S[4 * j + 2] = fmaf(da, S[4 * j + 2], w * bv.z);
            S[4 * j + 3] = fmaf(da, S[4 * j + 3], w * bv.w);
            acc = fmaf(S[4 * j + 0], cv.x, acc);
            a1 = fmaf(S[4 * j + 1], cv.y, a1);
            a2 = fmaf(S[4 * j + 2], cv.z, a2);
            a3 = fmaf(S[4 * j + 3], cv.w, a3);
          }
        }
        acc = (acc + a1) + (a2 + a3);
      } else {
#pragma unroll
        for (int i = 0; i < NPT; ++i) {
          const int n = l + 4 * i;
          if (n < N) {
            S[i] = fmaf(da, S[i], w * Bt[n]);
            acc = fmaf(S[i], Ct[n], acc);
          }
        }
      }
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      if (owner && l == 0) p.y[(size_t)(c0 + tk) * inner + h * p.Dv + col0 + pc] = fmaf(dskip, xv, acc);
    }
  }
  if (owner && to) {
#pragma unroll
    for (int i = 0; i < NPT; ++i) {
      const int n = VEC ? 16 * (i >> 2) + 4 * l + (i & 3) : l + 4 * i;
      if (n < N) to[n] = S[i];
    }
  }
  if (MODE == SSD_LOCAL && tid == 0 && col0 == 0) p.decay[row * p.H + h] = shrink;
}

// One thread per element of a request's matrices walks the run's chunks in order and writes what each begins with.
// Runs of one chunk are left alone.  The loads (four chunks' at a time) depend on no store.
__global__ void __launch_bounds__(256) ssd_carry_kernel(SsdArgs p) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.y;
  const size_t per = (size_t)p.H * p.Dv * p.N;
  const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= per) return;
  const int t0 = p.q_start[r], t1 = p.q_start[r + 1];
  if (t0 + p.chunk >= t1) return;
  const int h = (int)((unsigned)e / ((unsigned)p.Dv * (unsigned)p.N));
  const float* __restrict__ local = p.local;
  const float* __restrict__ decay = p.decay;
  float* __restrict__ carry = p.carry;
  float S = p.req_start[r] > 0 ? p.state[(size_t)p.slots[r] * p.slot_stride + e] : 0.f;
  const int nck = (t1 - t0 + p.chunk - 1) / p.chunk;
  const size_t row0 = (size_t)(r - p.row_off) + t0 / p.chunk;      // rows of one run follow one another
  int k = 0;
  for (; k + 4 < nck; k += 4) {
    float lo[4], de[4];
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      lo[x] = local[(row0 + k + x) * per + e];
      de[x] = decay[(row0 + k + x) * p.H + h];
    }
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      carry[(row0 + k + x) * per + e] = S;
      S = fmaf(de[x], S, lo[x]);
    }
  }
  for (; k < nck; ++k) {
    carry[(row0 + k) * per + e] = S;
    if (k + 1 < nck) S = fmaf(decay[(row0 + k) * p.H + h], S, local[(row0 + k) * per + e]);
  }
}

// Without chunks: cols, the value columns per block, shrink until the grid has about as many blocks as there are SMs.
// max_run: the step's longest run (chunked launches only: the grid's third extent).
KVB_EXPORT int kvb_ssd_scan(const SsdArgs* args, int R, int max_run, int dtype, cudaStream_t stream) {
  SsdArgs p = *args;
  if (R <= 0) return 0;
  if (p.H < 1 || p.G < 1 || p.H % p.G || p.N < 1 || p.N > 256 || p.Dv < 1 || R > 65535) return KVB_ERR_BAD_SIZE;
  int cols = p.Dv < 64 ? p.Dv : 64;
  unsigned nck = 1;
  if (p.chunk > 0) {
    if (!p.local || !p.carry || !p.decay || max_run < 1 || p.chunk % kSsdPiece) return KVB_ERR_BAD_SIZE;
    if ((long long)p.H * p.Dv * p.N > 0x7fffffffLL) return KVB_ERR_BAD_SIZE;
    nck = (unsigned)((max_run + p.chunk - 1) / p.chunk);
    if (nck > 65535) return KVB_ERR_BAD_SIZE;
  }
  while (cols > 8 && (long long)p.H * ((p.Dv + cols - 1) / cols) * R * nck < kvb_sm_count()) cols = (cols + 1) / 2;
  p.cols = cols;
  const int splits = (p.Dv + cols - 1) / cols;
  const int threads = (cols * 4 + 31) / 32 * 32;
  const size_t smem = ((size_t)kSsdPiece * (2 * p.N + cols) + 2 * kSsdPiece) * sizeof(float);
  const int npt = (p.N + 3) / 4;
  const dim3 grid(p.H * splits, R, nck);
#define KVB_SSD_MODE(NPT, MODE, VEC)                                                                                  \
  {                                                                                                                \
    if (smem > 48 * 1024) {                                                                                        \
      cudaError_t e = cudaFuncSetAttribute(ssd_scan_kernel<T, NPT, MODE, VEC>,                                     \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                \
      if (e != cudaSuccess) return (int)e;                                                                         \
    }                                                                                                              \
    kvb_launch(ssd_scan_kernel<T, NPT, MODE, VEC>, grid, dim3(threads), smem, stream, p);                          \
  }
#define KVB_SSD_VEC(MODE, VEC)                                                                                     \
  KVB_DISPATCH_DTYPE(dtype, T, {                                                                                   \
    if (npt <= 8) KVB_SSD_MODE(8, MODE, VEC)                                                                       \
    else if (npt <= 16) KVB_SSD_MODE(16, MODE, VEC)                                                                \
    else if (npt <= 32) KVB_SSD_MODE(32, MODE, VEC)                                                                \
    else KVB_SSD_MODE(64, MODE, VEC)                                                                               \
  })
#define KVB_SSD(MODE)                                                                                              \
  {                                                                                                                \
    if (p.N % 4 == 0) KVB_SSD_VEC(MODE, true) else KVB_SSD_VEC(MODE, false)                                        \
  }
  if (p.chunk > 0) {
    KVB_SSD(SSD_LOCAL);
    const size_t per = (size_t)p.H * p.Dv * p.N;
    kvb_launch(ssd_carry_kernel, dim3((unsigned)((per + 255) / 256), R), dim3(256), 0, stream, p);
    KVB_SSD(SSD_FINAL);
  } else {
    KVB_SSD(SSD_WHOLE);
  }
#undef KVB_SSD
#undef KVB_SSD_VEC
#undef KVB_SSD_MODE
  return kvb_launch_result();
}

// ---------------------------------------------------------------- gate, then a norm per group of channels
// y [T, width] float32; z [T, >= width] compute type with row stride ld_z; weight [width] float32.
// out[t, c] = v / sqrt(mean over c's group of v^2 + eps) * weight[c],  v = y * silu(z).
template <typename T>
__global__ void __launch_bounds__(256)
gated_group_norm_kernel(const float* __restrict__ y, const T* __restrict__ z, int ld_z, const float* __restrict__ weight,
                        T* __restrict__ out, int width, int groups, float eps) {
  __shared__ float part[8];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, grp = blockIdx.y;
  const int gs = width / groups, c0 = grp * gs;
  const float* yr = y + (size_t)t * width + c0;
  const T* zr = z + (size_t)t * ld_z + c0;
  float sq = 0.f;
  for (int i = threadIdx.x; i < gs; i += blockDim.x) {
    const float zv = to_f32(zr[i]);
    const float v = yr[i] * (zv * sigmoid_f(zv));
    sq = fmaf(v, v, sq);
  }
  sq = warp_sum(sq);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = sq;
  __syncthreads();
  float total = 0.f;
  for (int i = 0; i < (int)(blockDim.x >> 5); ++i) total += part[i];
  const float rstd = 1.0f / sqrtf(total / (float)gs + eps);
  for (int i = threadIdx.x; i < gs; i += blockDim.x) {
    const float zv = to_f32(zr[i]);
    const float v = yr[i] * (zv * sigmoid_f(zv));
    out[(size_t)t * width + c0 + i] = from_f32<T>(v * rstd * weight[c0 + i]);
  }
}

KVB_EXPORT int kvb_gated_group_norm(const float* y, const void* z, int ld_z, const float* weight, void* out, int T_,
                                    int width, int groups, float eps, int dtype, cudaStream_t stream) {
  if (T_ <= 0) return 0;
  if (groups < 1 || width < 1 || width % groups || groups > 65535) return KVB_ERR_BAD_SIZE;
  const int gs = width / groups;
  const int threads = gs >= 1024 ? 256 : (gs >= 256 ? 128 : 64);
  KVB_DISPATCH_DTYPE(dtype, T, (kvb_launch(gated_group_norm_kernel<T>, dim3(T_, groups), dim3(threads), 0, stream, y,
                                            (const T*)z, ld_z, weight, (T*)out, width, groups, eps)));
  return kvb_launch_result();
}
