// Mixers that carry a matrix state per head from token to token (the delta-rule family).
//
// Every member updates a state S [Dk, Dv] per head and token as
//     S <- diag(d) S - p (x^T S) + k c^T          (both products read the state before the token)
// and reads  o = S^T r  afterwards.  What differs between members is how d, p, x, k, c, r
// follow from the projections of the token:
//   * MODE_GENERAL: decay d = exp(-e^{-1/2} sigmoid(z_d + b_d)) per key channel, removal along
//     the unit key u = k / sqrt(|k|^2 + 1e-6) at the rate a = sigmoid(z_a + b_a):  p = a * u,
//     x = u, c = v, read-out by r.
//   * MODE_GATED: decay g = exp(-exp(A_h) softplus(z_d + b_d)) per key channel (or one per head), unit q and k
//     (q also times Dk^-1/2), write strength beta = sigmoid(z_b) per head; decaying first and
//     then correcting the state's prediction for k is the same update with d = g, p = beta k,
//     x = k * g, c = beta v, read-out by q.
// Columns of S are independent of each other, so a thread owns a quarter of one column (the
// key channels {i : (i / 4) % 4 == lane part}) in registers for the whole run of tokens.  With
// y = r * d the read-out is  o_j = y.s_j - (x.s_j)(p.r) + c_j (k.r)  over the state before the
// token, so one round of shuffles per token serves both the update and the read-out.
//
// A block owns the columns (or, when the grid would leave SMs idle, a share of the columns) of
// one (head, request): it walks the request's tokens of this step in chunks of 16.  A chunk is
// prepared (its projections become the float32 vectors above, one warp per token) and scanned
// (the threads that own the columns step through it and leave the read-outs in a float32
// scratch); up to eight more warps prepare chunk i + 1 while the scan walks chunk i, in two
// buffers, one block barrier per chunk.  A second small kernel norms each head's read-out (RMS,
// weight, sigmoid gate).  The scan is bound by shared memory: every column re-reads the token's
// five vectors, which is why a head's columns are spread over several SMs when there is room.  The state is read from the request's
// slot at the start (zero when the request starts at position 0) and written back at the end.
// Everything but the projections is float32.  A token's result does not depend on how the
// request was cut into steps: each token is prepared alone and the scan is sequential.
//
// Also here: the short causal convolution with SiLU in front of such a mixer, whose last
// inputs are part of the request's state.
#include "common.cuh"

enum DeltaMode { MODE_GENERAL = 0, MODE_GATED = 1 };

constexpr int kChunk = 16;

struct DeltaArgs {
  const void* r; int ld_r;          // read-out projection, [T, G * Dk] (q for MODE_GATED)
  const void* k; int ld_k;          // key projection, [T, G * Dk]
  const void* v; int ld_v;          // value projection, [T, H * Dv]
  const void* gate; int ld_gate;    // output gate before its sigmoid, [T, H * Dv]
  const void* decay; int ld_decay;  // z_d, [T, H * Dk]
  const void* aux; int ld_aux;      // MODE_GENERAL: z_a [T, H * Dk]; MODE_GATED: z_b [T, H]
  const float* decay_bias;          // b_d [H * Dk]
  const float* aux_bias;            // MODE_GENERAL: b_a [H * Dk]
  const float* head_rate;           // MODE_GATED: A [H]
  const float* norm_w;              // [H * Dv] or [Dv]
  int norm_per_head;
  float* state;                     // [slots, H, Dv, 4 KPL] at slot_stride floats per slot
  long long slot_stride;
  void* out; int ld_out;            // [T, H * Dv]
  const int* q_start;               // [R + 1] first token row of each request's run
  const int* req_start;             // [R] position of the run's first token
  const int* slots;                 // [R]
  int H, G, Dk, Dv;
  float eps;
  float* o_raw;                     // [T, H * Dv] float32 scratch: the read-outs before their norm
  int decay_per_head;               // MODE_GATED: z_d is [T, H] and b_d [H], one decay for all key channels of a head
  int gate_silu;                    // the output gate is silu(gate) instead of sigmoid(gate)
};

__device__ __forceinline__ float sigmoidf_(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplusf_(float z) { return z > 20.f ? z : log1pf(expf(z)); }

template <typename T, int KPL, int MODE>
__global__ void delta_scan_kernel(const DeltaArgs a, int n_scan, int cols_per_block) {
  constexpr int DKP = 4 * KPL;
  extern __shared__ float4 smem4[];
  float* smem = reinterpret_cast<float*>(smem4);
  pdl_trigger();
  pdl_wait();
  const int h = blockIdx.x, req = blockIdx.y;
  const int Dk = a.Dk, Dv = a.Dv;
  const int dvp = cols_per_block;                     // columns of this block (a multiple of 8), from col0 on
  const int col0 = blockIdx.z * cols_per_block;
  const int tok_floats = 5 * DKP + dvp + 4;           // d, p, x, k, y | c | (p.r, k.r)
  const int buf_floats = kChunk * tok_floats;
  const int t0 = a.q_start[req], t1 = a.q_start[req + 1];
  const int lane = threadIdx.x & 31;
  // The first n_scan threads own the columns; the others (if the block has any) prepare the
  // next chunk and finish the one before while the scan runs.
  const bool scanner = (int)threadIdx.x < n_scan;
  const int n_help = (int)blockDim.x - n_scan;
  const bool piped = n_help > 0;
  const int lcol = threadIdx.x >> 2, part = threadIdx.x & 3;     // column inside the block's share
  const int col = col0 + lcol;
  const bool owns = lcol < dvp && col < Dv;
  const int hk = h / (a.H / a.G);
  const T* rp = static_cast<const T*>(a.r);
  const T* kp = static_cast<const T*>(a.k);
  const T* vp = static_cast<const T*>(a.v);
  const T* dp = static_cast<const T*>(a.decay);
  const T* xp = static_cast<const T*>(a.aux);

  float s[KPL];
  float* my_state = a.state + (size_t)a.slots[req] * a.slot_stride + ((size_t)h * Dv + col) * DKP;
  const bool fresh = a.req_start[req] == 0;
#pragma unroll
  for (int e4 = 0; e4 < KPL / 4; ++e4) {
    float4 v4 = make_float4(0.f, 0.f, 0.f, 0.f);
    if (scanner && !fresh && owns) v4 = *reinterpret_cast<const float4*>(my_state + (e4 * 4 + part) * 4);
    s[e4 * 4 + 0] = v4.x; s[e4 * 4 + 1] = v4.y; s[e4 * 4 + 2] = v4.z; s[e4 * 4 + 3] = v4.w;
  }
  const float rate = MODE == MODE_GATED ? expf(a.head_rate[h]) : 0.60653065971263342f;   // e^{-1/2}
  const float q_scale = rsqrtf((float)Dk);

  // ---- a chunk's vectors, one warp per token (warps w0, w0 + nw, ... of the group that prepares)
  auto prepare = [&](int base, int n, float* buf, int w0, int nw, int th0, int nth) {
    constexpr int U = (DKP + 31) / 32;
    // A warp takes two tokens at a time and requests everything both need before it waits for any of it:
    // the time of a chunk's preparation is the latency of memory, not its amount.
    for (int c0 = w0; c0 < n; c0 += 2 * nw) {
      float kr_[2][U], rr_[2][U], zd_[2][U], za_[2][U], cv_[2][8], braw[2];
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int c = c0 + k * nw;
        const int t = base + (c < n ? c : c0);            // a missing second token reads the first again
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int i = u * 32 + lane;
          float kv = 0.f, rv = 0.f, zd = 0.f, za = 0.f;
          if (i < Dk) {
            kv = to_f32(kp[(size_t)t * a.ld_k + hk * Dk + i]);
            rv = to_f32(rp[(size_t)t * a.ld_r + hk * Dk + i]);
            const int di = a.decay_per_head ? h : h * Dk + i;
            zd = to_f32(dp[(size_t)t * a.ld_decay + di]) + a.decay_bias[di];
            if (MODE == MODE_GENERAL) za = to_f32(xp[(size_t)t * a.ld_aux + h * Dk + i]) + a.aux_bias[h * Dk + i];
          }
          kr_[k][u] = kv; rr_[k][u] = rv; zd_[k][u] = zd; za_[k][u] = za;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int j = u * 32 + lane;
          cv_[k][u] = (j < dvp && col0 + j < Dv) ? to_f32(vp[(size_t)t * a.ld_v + h * Dv + col0 + j]) : 0.f;
        }
        braw[k] = MODE == MODE_GATED ? to_f32(xp[(size_t)t * a.ld_aux + h]) : 0.f;
      }
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int c = c0 + k * nw;
        if (c >= n) continue;
        float* tok = buf + (size_t)c * tok_floats;
        float ksum = 0.f, rsum = 0.f;
#pragma unroll
        for (int u = 0; u < U; ++u) { ksum += kr_[k][u] * kr_[k][u]; rsum += rr_[k][u] * rr_[k][u]; }
        const float beta = MODE == MODE_GATED ? sigmoidf_(braw[k]) : 1.f;
        ksum = warp_sum(ksum);
        rsum = warp_sum(rsum);
        const float kinv = 1.0f / sqrtf(ksum + 1e-6f);
        const float rinv = MODE == MODE_GATED ? q_scale / sqrtf(rsum + 1e-6f) : 1.0f;
        float pr = 0.f, kr = 0.f;
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int i = u * 32 + lane;
          if (i >= DKP) continue;
          float d = 0.f, p = 0.f, x = 0.f, kk = 0.f, y = 0.f;
          if (i < Dk) {
            if (MODE == MODE_GENERAL) {
              const float unit = kr_[k][u] * kinv;
              const float rem = sigmoidf_(za_[k][u]);
              d = expf(-rate * sigmoidf_(zd_[k][u]));
              p = rem * unit; x = unit; kk = kr_[k][u]; y = rr_[k][u] * d;
              pr += p * rr_[k][u]; kr += kk * rr_[k][u];
            } else {
              const float kn = kr_[k][u] * kinv, qn = rr_[k][u] * rinv;
              d = expf(-rate * softplusf_(zd_[k][u]));
              p = beta * kn; x = kn * d; kk = kn; y = qn * d;
              kr += kn * qn;
            }
          }
          tok[i] = d; tok[DKP + i] = p; tok[2 * DKP + i] = x; tok[3 * DKP + i] = kk; tok[4 * DKP + i] = y;
        }
        pr = warp_sum(pr);
        kr = warp_sum(kr);
        if (MODE == MODE_GATED) pr = beta * kr;
        if (lane == 0) { tok[5 * DKP + dvp] = pr; tok[5 * DKP + dvp + 1] = kr; }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int j = u * 32 + lane;
          if (j < dvp) tok[5 * DKP + j] = MODE == MODE_GATED ? beta * cv_[k][u] : cv_[k][u];
        }
      }
    }
  };

  // ---- the scan over a chunk.  Every scanning thread takes part (the shuffles name the whole
  // warp); threads beyond the last column carry zeros and store nothing.
  auto scan = [&](int base, int n, const float* buf) {
    for (int c = 0; c < n; ++c) {        // unrolling by four was measured slower (3.2 against 2.6 ms for four layers)
      const float* tok = buf + (size_t)c * tok_floats;
      const float4* D4 = reinterpret_cast<const float4*>(tok);
      const float4* P4 = reinterpret_cast<const float4*>(tok + DKP);
      const float4* X4 = reinterpret_cast<const float4*>(tok + 2 * DKP);
      const float4* K4 = reinterpret_cast<const float4*>(tok + 3 * DKP);
      const float4* Y4 = reinterpret_cast<const float4*>(tok + 4 * DKP);
      // four partial sums per dot product: the chain of dependent additions is KPL / 4 long, not KPL
      float dx0 = 0.f, dx1 = 0.f, dx2 = 0.f, dx3 = 0.f, dy0 = 0.f, dy1 = 0.f, dy2 = 0.f, dy3 = 0.f;
#pragma unroll
      for (int e4 = 0; e4 < KPL / 4; ++e4) {
        const float4 xv = X4[e4 * 4 + part], yv = Y4[e4 * 4 + part];
        dx0 = fmaf(xv.x, s[e4 * 4 + 0], dx0); dx1 = fmaf(xv.y, s[e4 * 4 + 1], dx1);
        dx2 = fmaf(xv.z, s[e4 * 4 + 2], dx2); dx3 = fmaf(xv.w, s[e4 * 4 + 3], dx3);
        dy0 = fmaf(yv.x, s[e4 * 4 + 0], dy0); dy1 = fmaf(yv.y, s[e4 * 4 + 1], dy1);
        dy2 = fmaf(yv.z, s[e4 * 4 + 2], dy2); dy3 = fmaf(yv.w, s[e4 * 4 + 3], dy3);
      }
      float dx = (dx0 + dx1) + (dx2 + dx3), dy = (dy0 + dy1) + (dy2 + dy3);
      dx += __shfl_xor_sync(0xffffffffu, dx, 1); dy += __shfl_xor_sync(0xffffffffu, dy, 1);
      dx += __shfl_xor_sync(0xffffffffu, dx, 2); dy += __shfl_xor_sync(0xffffffffu, dy, 2);
      const float cj = lcol < dvp ? tok[5 * DKP + lcol] : 0.f;
      const float pr = tok[5 * DKP + dvp], kr = tok[5 * DKP + dvp + 1];
      if (part == 0 && owns) a.o_raw[(size_t)(base + c) * a.H * Dv + h * Dv + col] = dy - dx * pr + cj * kr;
#pragma unroll
      for (int e4 = 0; e4 < KPL / 4; ++e4) {
        const float4 dv = D4[e4 * 4 + part], pv = P4[e4 * 4 + part], kv = K4[e4 * 4 + part];
        s[e4 * 4 + 0] = fmaf(dv.x, s[e4 * 4 + 0], fmaf(kv.x, cj, -pv.x * dx));
        s[e4 * 4 + 1] = fmaf(dv.y, s[e4 * 4 + 1], fmaf(kv.y, cj, -pv.y * dx));
        s[e4 * 4 + 2] = fmaf(dv.z, s[e4 * 4 + 2], fmaf(kv.z, cj, -pv.z * dx));
        s[e4 * 4 + 3] = fmaf(dv.w, s[e4 * 4 + 3], fmaf(kv.w, cj, -pv.w * dx));
      }
    }
  };

  if (!piped) {
    // one group of threads prepares and scans in turn
    const int warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int base = t0; base < t1; base += kChunk) {
      const int n = min(kChunk, t1 - base);
      prepare(base, n, smem, warp, nwarps, threadIdx.x, blockDim.x);
      __syncthreads();
      scan(base, n, smem);
      __syncthreads();
    }
  } else {
    // Two buffers: in round i the scanning threads walk chunk i while the helpers prepare chunk i + 1.
    const int n_chunks = (t1 - t0 + kChunk - 1) / kChunk;
    const int hw = ((int)threadIdx.x - n_scan) >> 5, hnw = n_help >> 5, hth = (int)threadIdx.x - n_scan;
    if (!scanner && n_chunks > 0) prepare(t0, min(kChunk, t1 - t0), smem, hw, hnw, hth, n_help);
    __syncthreads();
    for (int i = 0; i < n_chunks; ++i) {
      const int base = t0 + i * kChunk;
      if (scanner) {
        scan(base, min(kChunk, t1 - base), smem + (size_t)(i & 1) * buf_floats);
      } else if (i + 1 < n_chunks) {
        prepare(base + kChunk, min(kChunk, t1 - base - kChunk), smem + (size_t)((i + 1) & 1) * buf_floats, hw, hnw, hth, n_help);
      }
      __syncthreads();
    }
  }
  if (scanner && owns) {
#pragma unroll
    for (int e4 = 0; e4 < KPL / 4; ++e4)
      *reinterpret_cast<float4*>(my_state + (e4 * 4 + part) * 4) =
          make_float4(s[e4 * 4 + 0], s[e4 * 4 + 1], s[e4 * 4 + 2], s[e4 * 4 + 3]);
  }
}

// Key channels per quarter column for a key size: the smallest of 4, 8, 16, 32 whose fourfold
// holds Dk (0: refused).  The state's rows are padded to four times this.
static int delta_kpl(int Dk) {
  for (int k = 4; k <= 32; k *= 2)
    if (4 * k >= Dk) return k;
  return 0;
}

KVB_EXPORT int kvb_delta_key_pad(int Dk) { return Dk >= 1 ? 4 * delta_kpl(Dk) : 0; }

// The read-outs' norm and gate: out[t, h, :] = o / sqrt(mean(o^2) + eps) * w * sigmoid(gate), one warp per (token, head).
template <typename T>
__global__ void delta_finish_kernel(const DeltaArgs a, int T_) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (unit >= (long long)T_ * a.H) return;
  const int t = (int)(unit / a.H), h = (int)(unit - (long long)t * a.H);
  const int Dv = a.Dv;
  const float* o = a.o_raw + (size_t)t * a.H * Dv + h * Dv;
  const T* gp = static_cast<const T*>(a.gate) + (size_t)t * a.ld_gate + h * Dv;
  T* outp = static_cast<T*>(a.out) + (size_t)t * a.ld_out + h * Dv;
  float ss = 0.f;
  for (int j = lane; j < Dv; j += 32) ss += o[j] * o[j];
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)Dv + a.eps);
  for (int j = lane; j < Dv; j += 32) {
    const float w = a.norm_w[(a.norm_per_head ? h * Dv : 0) + j];
    const float g = to_f32(gp[j]);
    outp[j] = from_f32<T>(o[j] * inv * w * (a.gate_silu ? g * sigmoidf_(g) : sigmoidf_(g)));
  }
}

template <typename T, int KPL, int MODE>
static int launch_scan(const DeltaArgs& a, int R, int T_, int max_run, cudaStream_t stream) {
  const int dv8 = (a.Dv + 7) & ~7;
  // A head's columns are shared out over several blocks while the grid would otherwise leave SMs idle (one
  // long prompt alone); shares are multiples of 8 columns.  The results do not depend on the split.
  int split = 1;
  // Never more blocks than SMs: two blocks on one SM take issue slots from each other's chain of dependent steps (32
  // heads in 256 blocks took 0.55 us a token, in 128 blocks 0.34).
  while ((long long)a.H * R * split * 2 <= kvb_sm_count() && dv8 / (split * 2) >= 8 && (dv8 / (split * 2)) % 8 == 0) split *= 2;
  const int cols = dv8 / split;
  const int n_scan = 4 * cols;
  static int max_threads = 0;                 // what the kernel's registers allow in one block
  if (max_threads == 0) {
    cudaFuncAttributes attr;
    cudaError_t e = cudaFuncGetAttributes(&attr, delta_scan_kernel<T, KPL, MODE>);
    if (e != cudaSuccess) return (int)e;
    max_threads = attr.maxThreadsPerBlock / 32 * 32;
  }
  if (n_scan > max_threads) return KVB_ERR_BAD_SIZE;
  // Up to eight warps beside the scanning ones prepare the next chunk (two tokens each) meanwhile.  Sixteen
  // were measured slower by half: the scan is a chain of dependent steps in two to eight warps, and every
  // further warp on the SM takes issue slots from them.
  int n_help = max_threads - n_scan < 256 ? max_threads - n_scan : 256;
  if (n_help < 128) n_help = 0;               // too few to keep up: the scanning threads do everything in turn
  if (max_run > 0 && max_run <= kChunk) n_help = 0;   // a single chunk per request (decode steps): nothing to overlap
  const size_t buf = (size_t)kChunk * (5 * 4 * KPL + cols + 4) * sizeof(float);
  const size_t smem = n_help ? 2 * buf : buf;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(delta_scan_kernel<T, KPL, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  kvb_launch(delta_scan_kernel<T, KPL, MODE>, dim3(a.H, R, split), dim3(n_scan + n_help), smem, stream, a, n_scan, cols);
  const long long units = (long long)T_ * a.H;
  kvb_launch(delta_finish_kernel<T>, dim3((unsigned)((units + 7) / 8)), dim3(256), 0, stream, a, T_);
  return kvb_launch_result();
}

template <typename T, int MODE>
static int launch_scan_kpl(const DeltaArgs& a, int R, int T_, int max_run, cudaStream_t stream) {
  switch (delta_kpl(a.Dk)) {
    case 4: return launch_scan<T, 4, MODE>(a, R, T_, max_run, stream);
    case 8: return launch_scan<T, 8, MODE>(a, R, T_, max_run, stream);
    case 16: return launch_scan<T, 16, MODE>(a, R, T_, max_run, stream);
    case 32: return launch_scan<T, 32, MODE>(a, R, T_, max_run, stream);
  }
  return KVB_ERR_BAD_SIZE;
}

// max_run: the longest run of tokens among the requests if the host knows it (0: unknown); the
// results do not depend on it.  Refuses: Dk > 128, Dv > 256, Dv > 128 together with Dk > 64 (a
// thread's quarter column would not stay in registers), heads that do not group evenly.
KVB_EXPORT int kvb_delta_scan(const DeltaArgs* args, int mode, int R, int T_, int max_run, int dtype, cudaStream_t stream) {
  const DeltaArgs& a = *args;
  if (R <= 0 || T_ <= 0) return 0;
  if (a.o_raw == nullptr) return KVB_ERR_BAD_SIZE;
  if (a.Dk < 1 || a.Dk > 128 || a.Dv < 1 || a.Dv > 256 || (a.Dk > 64 && a.Dv > 128)) return KVB_ERR_BAD_SIZE;
  if (a.G < 1 || a.H % a.G || R > 65535) return KVB_ERR_BAD_SIZE;
  if (mode != MODE_GENERAL && mode != MODE_GATED) return KVB_ERR_BAD_SIZE;
  if (mode == MODE_GENERAL) {
    KVB_DISPATCH_DTYPE(dtype, T, return (launch_scan_kpl<T, MODE_GENERAL>(a, R, T_, max_run, stream)));
  } else {
    KVB_DISPATCH_DTYPE(dtype, T, return (launch_scan_kpl<T, MODE_GATED>(a, R, T_, max_run, stream)));
  }
  return KVB_ERR_BAD_DTYPE;
}

// ---------------------------------------------------------------- short causal convolution + SiLU
// out[t, c] = silu( sum_j w[c, j] * in[p - (taps - 1) + j, c] ), p the token's position: the last
// column of w weighs the token itself, inputs before position 0 are zero, and inputs before the
// step's run come from the request's tail (its last taps - 1 inputs, tail[j] holding position
// start - (taps - 1) + j).
template <typename T>
__device__ __forceinline__ float conv_input(const T* in, int ld, const float* tail, int C, int c, int sp, int start,
                                            int row0, int taps) {
  if (sp < 0) return 0.f;
  if (sp >= start) return to_f32(in[(size_t)(row0 + sp - start) * ld + c]);
  return tail[(size_t)(sp - (start - (taps - 1))) * C + c];
}

template <typename T>
__global__ void conv_silu_kernel(const T* __restrict__ in, int ld, const float* __restrict__ w, int taps,
                                 const float* __restrict__ tails, long long slot_stride, T* __restrict__ out, int C,
                                 const int* __restrict__ positions, const int* __restrict__ token_req,
                                 const int* __restrict__ q_start, const int* __restrict__ req_start,
                                 const int* __restrict__ slots, int act, const float* __restrict__ in_bias,
                                 const float* __restrict__ out_bias) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int pos = positions[t], r = token_req[t];
  const int start = req_start[r], row0 = q_start[r];
  const float* tail = tails + (size_t)slots[r] * slot_stride;
  const float ib = in_bias ? in_bias[c] : 0.f;      // joins every input that exists (not the zeros before the start)
  float acc = out_bias ? out_bias[c] : 0.f;
  for (int j = 0; j < taps; ++j) {
    const int sp = pos - (taps - 1) + j;
    if (sp < 0) continue;
    acc = fmaf(w[(size_t)c * taps + j], conv_input(in, ld, tail, C, c, sp, start, row0, taps) + ib, acc);
  }
  out[(size_t)t * C + c] = from_f32<T>(act == 0 ? acc / (1.0f + expf(-acc)) : acc);
}

// The same for rows of channels that are multiples of 16 bytes: a thread takes VEC consecutive channels of one
// token (one 16-byte load per tap).  It can also write the convolved keys and values of an attention mixer into
// the request's pages, whose rows hold [key | value] per token and key/value head (`ap.pages` not null): the
// channels from k_off on are kv_heads keys of Dk, those from v_off on kv_heads values of Dv.
struct AppendArgs {
  void* pages; const int* block_table; int max_pages, page_size, num_pages, k_off, v_off, kv_heads, Dk, Dv; int* status;
};

template <typename T> struct Vec16;
template <> struct Vec16<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float* x) {
    const float4 u = *reinterpret_cast<const float4*>(p); x[0] = u.x; x[1] = u.y; x[2] = u.z; x[3] = u.w;
  }
  static __device__ __forceinline__ void store(float* p, const float* x) {
    *reinterpret_cast<float4*>(p) = make_float4(x[0], x[1], x[2], x[3]);
  }
};
template <> struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* x) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const unsigned w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) { x[2 * e] = __uint_as_float(w[e] << 16); x[2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u); }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* x) {
    unsigned w[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      __nv_bfloat162 v = __floats2bfloat162_rn(x[2 * e], x[2 * e + 1]);
      w[e] = *reinterpret_cast<unsigned*>(&v);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  }
};

// TAPS > 0: the number of taps, known when the kernel is built; the thread's VEC x TAPS weights are then fetched with
// 16-byte loads into registers.  TAPS 0: any number, the weights fetched one by one.
template <typename T, int TAPS>
__global__ void conv_vec_kernel(const T* __restrict__ in, int ld, const float* __restrict__ w, int taps,
                                const float* __restrict__ tails, long long slot_stride, T* __restrict__ out, int C,
                                int T_, const int* __restrict__ positions, const int* __restrict__ token_req,
                                const int* __restrict__ q_start, const int* __restrict__ req_start,
                                const int* __restrict__ slots, int act, AppendArgs ap,
                                const float* __restrict__ in_bias, const float* __restrict__ out_bias) {
  constexpr int VEC = Vec16<T>::N;
  pdl_trigger();
  pdl_wait();
  const int groups = C / VEC;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)T_ * groups) return;
  const int t = (int)(idx / groups), c = (int)(idx - (long long)t * groups) * VEC;
  const int pos = positions[t], r = token_req[t];
  // A request's tokens of this step are consecutive rows: the input `back` tokens back is row t - back when that row
  // belongs to the same request, which one look at token_req tells; only the first taps - 1 tokens of a run go on to
  // the request's tail (and look up where it lies).
  auto older = [&](int back, float* x) {
    const int sp = pos - back;
    if (sp < 0) {
#pragma unroll
      for (int e = 0; e < VEC; ++e) x[e] = 0.f;
      return;
    }
    const int start = req_start[r];
    const float* tp = tails + (size_t)slots[r] * slot_stride + (size_t)(sp - (start - (taps - 1))) * C + c;
#pragma unroll
    for (int e = 0; e < VEC; ++e) x[e] = tp[e];
  };
  float acc[VEC], ib[VEC];
#pragma unroll
  for (int e = 0; e < VEC; ++e) {
    acc[e] = out_bias ? out_bias[c + e] : 0.f;
    ib[e] = in_bias ? in_bias[c + e] : 0.f;         // joins every input that exists (not the zeros before the start)
  }
  if (TAPS > 0) {
    constexpr int NT = TAPS > 0 ? TAPS : 1;
    float wv[VEC * NT];                       // channel e's taps at wv[e * NT ..]; c * NT floats is a multiple of 16 bytes
#pragma unroll
    for (int i = 0; i < VEC * NT; i += 4) {
      const float4 u = *reinterpret_cast<const float4*>(w + (size_t)c * NT + i);
      wv[i] = u.x; wv[i + 1] = u.y; wv[i + 2] = u.z; wv[i + 3] = u.w;
    }
    bool same[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      const int back = NT - 1 - j;
      same[j] = back == 0 || (t - back >= 0 && token_req[t - back] == r);
    }
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      const int back = NT - 1 - j;
      float x[VEC];
      if (same[j]) Vec16<T>::load(in + (size_t)(t - back) * ld + c, x);
      else older(back, x);
      if (pos - back >= 0) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) x[e] += ib[e];
      }
#pragma unroll
      for (int e = 0; e < VEC; ++e) acc[e] = fmaf(wv[e * NT + j], x[e], acc[e]);
    }
  } else {
    for (int j = 0; j < taps; ++j) {
      const int back = taps - 1 - j;
      float x[VEC];
      if (back == 0 || (t - back >= 0 && token_req[t - back] == r)) Vec16<T>::load(in + (size_t)(t - back) * ld + c, x);
      else older(back, x);
      if (pos - back >= 0) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) x[e] += ib[e];
      }
#pragma unroll
      for (int e = 0; e < VEC; ++e) acc[e] = fmaf(w[(size_t)(c + e) * taps + j], x[e], acc[e]);
    }
  }
  if (act == 0) {
#pragma unroll
    for (int e = 0; e < VEC; ++e) acc[e] = acc[e] / (1.0f + expf(-acc[e]));
  }
  Vec16<T>::store(out + (size_t)t * C + c, acc);
  if (ap.pages != nullptr && c >= ap.k_off) {
    const bool is_v = c >= ap.v_off;
    const int width = is_v ? ap.Dv : ap.Dk;
    const int rel = c - (is_v ? ap.v_off : ap.k_off);
    const int g = rel / width, i = rel - g * width;
    if (g < ap.kv_heads) {
      const int lp = pos / ap.page_size;
      const int page = lp < ap.max_pages ? ap.block_table[(size_t)r * ap.max_pages + lp] : -1;
      if (page < 0 || page >= ap.num_pages) {
        atomicCAS(ap.status, 0, KVB_STATUS_UNMAPPED_PAGE);
      } else {
        T* row = static_cast<T*>(ap.pages) +
                 (((size_t)page * ap.kv_heads + g) * ap.page_size + (pos % ap.page_size)) * (ap.Dk + ap.Dv);
        Vec16<T>::store(row + (is_v ? ap.Dk : 0) + i, acc);
      }
    }
  }
}

// After the convolution: the request's tail becomes the last taps - 1 inputs up to the end of the
// step's run (older ones move up when the run is shorter than the tail).
constexpr int kMaxTail = 15;
template <typename T>
__global__ void conv_tail_kernel(const T* __restrict__ in, int ld, int taps, float* __restrict__ tails,
                                 long long slot_stride, int C, const int* __restrict__ q_start,
                                 const int* __restrict__ req_start, const int* __restrict__ ctx_len,
                                 const int* __restrict__ slots) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int start = req_start[r], row0 = q_start[r], end = ctx_len[r];
  float* tail = tails + (size_t)slots[r] * slot_stride;
  float keep[kMaxTail];
#pragma unroll
  for (int j = 0; j < kMaxTail; ++j)
    if (j < taps - 1) keep[j] = conv_input(in, ld, tail, C, c, end - (taps - 1) + j, start, row0, taps);
#pragma unroll
  for (int j = 0; j < kMaxTail; ++j)
    if (j < taps - 1) tail[(size_t)j * C + c] = keep[j];
}

// append: null, or where the convolved keys and values of an attention mixer go as well (see AppendArgs; only rows
// of whole 16-byte groups can: the launcher refuses otherwise and the caller writes them with a kernel of its own).
// in: [T, >= C] with row stride ld; w [C, taps] float32; tails: the tail of slot 0, slot_stride
// floats from slot to slot, each [taps - 1, C]; out [T, C] dense.  act: 0 SiLU behind the sum, 1 the
// bare sum.  in_bias (float32 [C] or null) joins every input before it is weighed (the inputs before a
// sequence's start stay zero; the tails keep the inputs without it), out_bias (float32 [C] or null) joins
// the sum.  Refuses taps > 16.
KVB_EXPORT int kvb_conv_silu(const void* in, int ld, const float* w, int taps, float* tails, long long slot_stride,
                             void* out, int C, int T_, int R, const int* positions, const int* token_req,
                             const int* q_start, const int* req_start, const int* ctx_len, const int* slots,
                             int act, const AppendArgs* append, const float* in_bias, const float* out_bias, int dtype,
                             cudaStream_t stream) {
  if (T_ <= 0 || R <= 0) return 0;
  if (taps < 1 || taps - 1 > kMaxTail || C < 1 || act < 0 || act > 1) return KVB_ERR_BAD_SIZE;
  const int threads = 128;
  const int by = (C + threads - 1) / threads;
  // rows of whole 16-byte groups: the vector form, which can also write keys and values into their pages
  const int vec = dtype == KVB_F32 ? 4 : 8;
  AppendArgs ap = {};
  if (append != nullptr) ap = *append;
  const bool aligned = C % vec == 0 && ld % vec == 0 && ((uintptr_t)in % 16) == 0 && ((uintptr_t)out % 16) == 0;
  if (ap.pages != nullptr &&
      !(aligned && ap.Dk % vec == 0 && ap.Dv % vec == 0 && ap.k_off % vec == 0 && ap.v_off % vec == 0 &&
        ((uintptr_t)ap.pages % 16) == 0 && ap.kv_heads >= 1 && ap.page_size >= 1 &&
        ap.k_off + ap.kv_heads * ap.Dk <= ap.v_off && ap.v_off + ap.kv_heads * ap.Dv <= C))
    return KVB_ERR_BAD_SIZE;
  if (aligned) {
    const long long units = (long long)T_ * (C / vec);
    const bool w16 = ((uintptr_t)w % 16) == 0;
#define KVB_CONV(TAPS)                                                                                                  \
  kvb_launch(conv_vec_kernel<T, TAPS>, dim3((unsigned)((units + 255) / 256)), dim3(256), 0, stream, (const T*)in, ld, w, \
             taps, (const float*)tails, slot_stride, (T*)out, C, T_, positions, token_req, q_start, req_start, slots, act, ap, \
             in_bias, out_bias)
    KVB_DISPATCH_DTYPE(dtype, T, {
      if (taps == 2 && w16) KVB_CONV(2);
      else if (taps == 3 && w16) KVB_CONV(3);
      else if (taps == 4 && w16) KVB_CONV(4);
      else KVB_CONV(0);
      if (taps > 1)
        kvb_launch(conv_tail_kernel<T>, dim3(R, by), dim3(threads), 0, stream, (const T*)in, ld, taps, tails, slot_stride,
                   C, q_start, req_start, ctx_len, slots);
    });
#undef KVB_CONV
    return kvb_launch_result();
  }
  KVB_DISPATCH_DTYPE(dtype, T, {
    kvb_launch(conv_silu_kernel<T>, dim3(T_, by), dim3(threads), 0, stream, (const T*)in, ld, w, taps,
               (const float*)tails, slot_stride, (T*)out, C, positions, token_req, q_start, req_start, slots, act, in_bias,
               out_bias);
    if (taps > 1)
      kvb_launch(conv_tail_kernel<T>, dim3(R, by), dim3(threads), 0, stream, (const T*)in, ld, taps, tails, slot_stride,
                 C, q_start, req_start, ctx_len, slots);
  });
  return kvb_launch_result();
}
